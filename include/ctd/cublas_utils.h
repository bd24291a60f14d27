// The reference keeps a process-wide cuBLAS handle here (emberlm include/ctd/cublas_utils.h). This
// build has no cuBLAS underneath: every GEMM is a ctdk kernel (ctdk_gemm). The header exists so that
// code which merely includes it still compiles; it declares nothing.
#pragma once
#include "b200/core.hpp"
