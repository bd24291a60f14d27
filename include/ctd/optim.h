// SGD, ParamGroup, AdamW, clip_grad_norm_: see b200/optim.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/optim.hpp"
