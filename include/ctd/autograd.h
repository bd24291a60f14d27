// the autograd tape: Node, Edge, AutogradMeta, NoGradGuard, checkpoint, ...: see b200/core.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/core.hpp"
