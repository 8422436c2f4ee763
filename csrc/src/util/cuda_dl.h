// CUDA driver and NVML entry points resolved at run time, so that the host
// library also loads on a machine without a GPU or driver (the host-memory heap
// back end and the bootstrap need neither).  `cu()` returns the table or null
// when libcuda.so.1 is missing (reference: src/host/init/cudawrap.cpp, nvmlwrap.cpp).
#pragma once
#include <cuda.h>

#include <string>

namespace bshmem {

#define BSHMEM_CU_FUNCS(X)              \
  X(cuInit)                             \
  X(cuGetErrorString)                   \
  X(cuDriverGetVersion)                 \
  X(cuDeviceGet)                        \
  X(cuDeviceGetCount)                   \
  X(cuDeviceGetAttribute)               \
  X(cuDeviceGetName)                    \
  X(cuDeviceGetUuid)                    \
  X(cuDeviceGetPCIBusId)                \
  X(cuDeviceCanAccessPeer)              \
  X(cuDeviceGetP2PAttribute)            \
  X(cuCtxGetCurrent)                    \
  X(cuCtxSetCurrent)                    \
  X(cuCtxGetDevice)                     \
  X(cuDevicePrimaryCtxRetain)           \
  X(cuDevicePrimaryCtxRelease)          \
  X(cuMemGetAllocationGranularity)      \
  X(cuMemAddressReserve)                \
  X(cuMemAddressFree)                   \
  X(cuMemCreate)                        \
  X(cuMemRelease)                       \
  X(cuMemMap)                           \
  X(cuMemUnmap)                         \
  X(cuMemSetAccess)                     \
  X(cuMemExportToShareableHandle)       \
  X(cuMemImportFromShareableHandle)     \
  X(cuMemGetAllocationPropertiesFromHandle) \
  X(cuMemRetainAllocationHandle)        \
  X(cuMemGetAddressRange)               \
  X(cuMulticastCreate)                  \
  X(cuMulticastAddDevice)               \
  X(cuMulticastBindMem)                 \
  X(cuMulticastUnbind)                  \
  X(cuMulticastGetGranularity)          \
  X(cuStreamWriteValue64)               \
  X(cuStreamWaitValue64)                \
  X(cuStreamWriteValue32)               \
  X(cuStreamWaitValue32)                \
  X(cuPointerGetAttribute)              \
  X(cuModuleGetGlobal)                  \
  X(cuTensorMapEncodeTiled)

struct CuTable {
#define X(name) decltype(&::name) name##_ = nullptr;
  BSHMEM_CU_FUNCS(X)
#undef X
};

// Null when the driver library cannot be loaded.  Missing individual symbols
// are left null and reported by `missing`.
const CuTable* cu(std::string* missing = nullptr);
std::string cu_error_string(CUresult r);

#define CU_CHECK_RET(call, retval)                                                    \
  do {                                                                                \
    CUresult _r = (call);                                                             \
    if (_r != CUDA_SUCCESS) {                                                         \
      ERROR_PRINT("%s failed: %s", #call, ::bshmem::cu_error_string(_r).c_str());     \
      return retval;                                                                  \
    }                                                                                 \
  } while (0)

// ---- NVML (optional; only used to describe the NVLink fabric) ----
struct NvlinkInfo {
  bool nvml_loaded = false;
  int active_links = 0;       // links of this GPU that report an active state
  int link_version = 0;       // NVLink generation reported by NVML
  bool all_links_to_switch = false;
  std::string driver_version;
};
NvlinkInfo nvml_probe_nvlink(const char* pci_bus_id);

}  // namespace bshmem
