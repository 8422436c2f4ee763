// Every PE writes its number into its right-hand neighbour with a single-element put issued from a kernel.
//   python -m nvshmem_b200.launch -n 4 -- examples/bin/dev-guide-ring
// (counterpart of the reference's examples/dev-guide-ring.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

__global__ void write_to_neighbour(int* slot) {
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  nvshmem_int_p(slot, me, (me + 1) % n);
}

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  int* slot = (int*)nvshmem_malloc(sizeof(int));
  write_to_neighbour<<<1, 1, 0, stream>>>(slot);
  nvshmemx_barrier_all_on_stream(stream);  // the put of my left-hand neighbour has landed
  int got = -1;
  cudaMemcpyAsync(&got, slot, sizeof(int), cudaMemcpyDeviceToHost, stream);
  cudaStreamSynchronize(stream);
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes(), want = (me + n - 1) % n;
  printf("PE %d received %d (%s)\n", me, got, got == want ? "ok" : "WRONG");
  nvshmem_free(slot);
  nvshmem_finalize();
  return got == want ? 0 : 1;
}
