// TensorDict, load_safetensors, save_safetensors: see b200/io.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/io.hpp"
