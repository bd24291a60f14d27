// nn::RMSNorm: see b200/nn.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/nn.hpp"
