// rms_norm and its backward: see b200/ops.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/ops.hpp"
