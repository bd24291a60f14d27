// nn::LlamaConfig, the presets, nn::Model, nn::build_model: see b200/nn.hpp (one header per group of the ctd:: surface).
#pragma once
#include "../b200/nn.hpp"
#include "../b200/io.hpp"
