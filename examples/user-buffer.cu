// Memory that the application allocated itself (CUDA virtual memory management: cuMemCreate + cuMemMap)
// becomes symmetric: nvshmemx_buffer_register_symmetric maps it into every PE's view of the heap and
// returns its symmetric address, which then works with every RMA and collective call.
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/user-buffer
// (counterpart of the reference's examples/user-buffer.cu)
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include "nvshmem.h"
#include "nvshmemx.h"

constexpr size_t BYTES = 512ul << 20;  // a multiple of the heap's growth granule
constexpr size_t NELEMS = 2048;

__global__ void init_data(float* x, size_t n, float base) {
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] = base + (float)i;
}

#define CU_OK(call)                                                        \
  do {                                                                     \
    CUresult r_ = (call);                                                  \
    if (r_ != CUDA_SUCCESS) {                                              \
      fprintf(stderr, "%s:%d: driver error %d\n", __FILE__, __LINE__, r_); \
      exit(1);                                                             \
    }                                                                      \
  } while (0)

int main() {
  nvshmem_init();
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  const int dev = nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE);
  cudaSetDevice(dev);
  cudaFree(0);

  // The application's own allocation: local to this GPU, shareable as a file descriptor.
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle handle;
  CUdeviceptr user = 0;
  CU_OK(cuMemCreate(&handle, BYTES, &prop, 0));
  CU_OK(cuMemAddressReserve(&user, BYTES, 0, 0, 0));
  CU_OK(cuMemMap(user, BYTES, 0, handle, 0));
  CUmemAccessDesc acc = {};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU_OK(cuMemSetAccess(user, BYTES, &acc, 1));

  float* sym = (float*)nvshmemx_buffer_register_symmetric((void*)user, BYTES, 0);
  if (!sym) {
    fprintf(stderr, "PE %d: registration failed\n", me);
    return 1;
  }
  float* source = sym;
  float* dest = sym + NELEMS;
  init_data<<<8, 256>>>(source, NELEMS, (float)(me * 10000));
  cudaMemset(dest, 0, NELEMS * sizeof(float));
  nvshmemx_barrier_all_on_stream(0);
  // Both sides of this put live in registered user memory.
  nvshmemx_float_put_on_stream(dest, source, NELEMS, (me + 1) % n, 0);
  nvshmemx_barrier_all_on_stream(0);
  float* host = (float*)malloc(NELEMS * sizeof(float));
  cudaMemcpy(host, dest, NELEMS * sizeof(float), cudaMemcpyDeviceToHost);
  const float base = (float)(((me + n - 1) % n) * 10000);
  size_t bad = 0;
  for (size_t i = 0; i < NELEMS; ++i) bad += host[i] != base + (float)i;
  // The caller's own mapping aliases the same memory.
  float first = -1.f;
  cudaMemcpy(&first, (void*)(user + NELEMS * sizeof(float)), sizeof(float), cudaMemcpyDeviceToHost);
  printf("PE %d: put through registered memory, %zu wrong; alias reads %.0f (expects %.0f)\n", me, bad, first, base);
  int st = nvshmemx_buffer_unregister_symmetric(sym, BYTES);
  CU_OK(cuMemUnmap(user, BYTES));
  CU_OK(cuMemAddressFree(user, BYTES));
  CU_OK(cuMemRelease(handle));
  free(host);
  nvshmem_finalize();
  return bad != 0 || first != base || st != 0;
}
