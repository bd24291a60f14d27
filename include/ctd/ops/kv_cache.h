// write_kv_inplace, read_kv_expanded: see b200/ops.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/ops.hpp"
