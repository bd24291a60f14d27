// CTD_CUDA_CHECK, CTD_CUDA_CHECK_KERNEL: see b200/core.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/core.hpp"
