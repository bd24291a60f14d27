// Allocator, cuda_allocator, cpu_allocator, pinned_cpu_allocator, allocator_for: see b200/core.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/core.hpp"
