// A kernel that synchronises with the other PEs from the device has to be co-resident on every GPU:
// nvshmemx_collective_launch checks that and launches it cooperatively.
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/collective-launch
// (counterpart of the reference's examples/collective-launch.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

__global__ void reduce_ring(int* target, int npes) {
  const int me = nvshmem_my_pe();
  const int peer = (me + 1) % npes;
  int value = me;
  for (int round = 1; round < npes; ++round) {
    nvshmem_int_p(target, value, peer);
    nvshmem_barrier_all();  // device-side barrier: every PE's kernel must be running
    value = *target + me;
    nvshmem_barrier_all();
  }
  *target = value;
}

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  int npes = nvshmem_n_pes(), me = nvshmem_my_pe();
  int* target = (int*)nvshmem_calloc(1, sizeof(int));
  void* args[] = {&target, &npes};
  int max_grid = 0;
  nvshmemx_collective_launch_query_gridsize((const void*)reduce_ring, dim3(1), args, 0, &max_grid);
  int st = nvshmemx_collective_launch((const void*)reduce_ring, dim3(1), dim3(1), args, 0, 0);
  cudaDeviceSynchronize();
  int got = 0;
  cudaMemcpy(&got, target, sizeof(int), cudaMemcpyDeviceToHost);
  // After npes-1 rounds of "take the left neighbour's running sum and add my rank" every PE holds 0+1+...+npes-1.
  const int want = npes * (npes - 1) / 2;
  printf("PE %d: co-resident grid limit %d, launch status %d, sum %d (%s)\n", me, max_grid, st, got, got == want ? "ok" : "WRONG");
  nvshmem_free(target);
  nvshmem_finalize();
  return st == 0 && got == want ? 0 : 1;
}
