// Umbrella header: host API for every translation unit, device API in addition
// for CUDA translation units (reference: src/include/nvshmem.h).
#pragma once
#include "nvshmem_host.h"
#ifdef __CUDACC__
#include "bshmem/device_api.cuh"
#include "bshmem/tile.cuh"
#endif
