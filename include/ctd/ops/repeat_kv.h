// repeat_kv_heads, repeat_kv_sum_impl, mul_scalar: see b200/ops.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/ops.hpp"
