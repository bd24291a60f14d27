// Storage, StoragePtr, make_storage: see b200/core.hpp (one header per group of the ctd:: surface).
#pragma once
#include "b200/core.hpp"
