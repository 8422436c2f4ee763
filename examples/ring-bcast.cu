// PE 0's data travels round the ring: each PE waits for a signal, forwards data and signal to the next
// PE (put, fence, signal), and the last one stops.
//   python -m nvshmem_b200.launch -n 4 -- examples/bin/ring-bcast
// (counterpart of the reference's examples/ring-bcast.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

__global__ void ring_bcast(int* data, size_t nelem, int root, uint64_t* psync) {
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  const int peer = (me + 1) % n;
  if (me == root) *psync = 1;
  nvshmem_signal_wait_until(psync, NVSHMEM_CMP_NE, 0);
  if (me == root) *psync = 0;
  if (peer == root) return;  // the ring is closed
  nvshmem_int_put(data, data, nelem, peer);
  nvshmem_fence();  // the data is ordered before the signal at the same PE
  nvshmemx_signal_op(psync, 1, NVSHMEM_SIGNAL_SET, peer);
  *psync = 0;
}

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  const int me = nvshmem_my_pe();
  const size_t n = 32;
  int* data = (int*)nvshmem_malloc(n * sizeof(int));
  uint64_t* psync = (uint64_t*)nvshmem_calloc(1, sizeof(uint64_t));
  int host[32];
  for (size_t i = 0; i < n; ++i) host[i] = me == 0 ? (int)i : -1;
  cudaMemcpy(data, host, n * sizeof(int), cudaMemcpyHostToDevice);
  int root = 0;
  size_t nelem = n;
  nvshmem_barrier_all();
  void* args[] = {&data, &nelem, &root, &psync};
  nvshmemx_collective_launch((const void*)ring_bcast, dim3(1), dim3(1), args, 0, 0);
  cudaDeviceSynchronize();
  nvshmem_barrier_all();
  cudaMemcpy(host, data, n * sizeof(int), cudaMemcpyDeviceToHost);
  int bad = 0;
  for (size_t i = 0; i < n; ++i) bad += host[i] != (int)i;
  printf("PE %d: ring broadcast, %d wrong\n", me, bad);
  nvshmem_free(data);
  nvshmem_free(psync);
  nvshmem_finalize();
  return bad != 0;
}
