// mse_loss, cross_entropy, cross_entropy_masked: see b200/ops.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/ops.hpp"
