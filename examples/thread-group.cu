// Block-scoped collective from inside a kernel: all threads of the CTA call fcollect together.
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/thread-group
// (counterpart of the reference's examples/thread-group.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

constexpr int NELEMS = 1024;

__global__ void gather(int* dst, const int* src) { nvshmemx_int_fcollect_block(NVSHMEM_TEAM_WORLD, dst, src, NELEMS); }

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  int* src = (int*)nvshmem_malloc(NELEMS * sizeof(int));
  int* dst = (int*)nvshmem_malloc((size_t)NELEMS * n * sizeof(int));
  int* host = new int[(size_t)NELEMS * n];
  for (int i = 0; i < NELEMS; ++i) host[i] = me * NELEMS + i;
  cudaMemcpy(src, host, NELEMS * sizeof(int), cudaMemcpyHostToDevice);
  nvshmem_barrier_all();
  void* args[] = {&dst, &src};
  nvshmemx_collective_launch((const void*)gather, dim3(1), dim3(256), args, 0, 0);
  cudaDeviceSynchronize();
  cudaMemcpy(host, dst, (size_t)NELEMS * n * sizeof(int), cudaMemcpyDeviceToHost);
  int bad = 0;
  for (int i = 0; i < NELEMS * n; ++i) bad += host[i] != i;
  printf("PE %d: fcollect_block of %d x %d ints, %d wrong\n", me, n, NELEMS, bad);
  delete[] host;
  nvshmem_free(src);
  nvshmem_free(dst);
  nvshmem_finalize();
  return bad != 0;
}
