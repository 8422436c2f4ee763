// Extension API header; everything lives in nvshmem.h (reference: src/include/nvshmemx.h).
#pragma once
#include "nvshmem.h"
