// RopeScaling, rope, apply_rope_inplace: see b200/ops.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/ops.hpp"
