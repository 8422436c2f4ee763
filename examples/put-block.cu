// One CTA moves a large block to the next PE with a block-scoped put (all threads share the copy).
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/put-block
// (counterpart of the reference's examples/put-block.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

constexpr size_t N = 1 << 20;

__global__ void fill(int* x, int base) {
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (size_t)gridDim.x * blockDim.x) x[i] = base + (int)i;
}
__global__ void send(int* dst, const int* src, int peer) {
  const size_t per = N / gridDim.x;
  nvshmemx_int_put_block(dst + blockIdx.x * per, src + blockIdx.x * per, per, peer);
}
__global__ void verify(const int* x, int base, int* bad) {
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (size_t)gridDim.x * blockDim.x)
    if (x[i] != base + (int)i) atomicAdd(bad, 1);
}

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  int* src = (int*)nvshmem_malloc(N * sizeof(int));
  int* dst = (int*)nvshmem_malloc(N * sizeof(int));
  int* bad;
  cudaMalloc(&bad, sizeof(int));
  cudaMemset(bad, 0, sizeof(int));
  fill<<<128, 256>>>(src, me * 1000);
  nvshmemx_barrier_all_on_stream(0);
  send<<<16, 512>>>(dst, src, (me + 1) % n);
  nvshmemx_barrier_all_on_stream(0);  // completes the puts and tells the receiver
  verify<<<128, 256>>>(dst, ((me + n - 1) % n) * 1000, bad);
  int h_bad = -1;
  cudaMemcpy(&h_bad, bad, sizeof(int), cudaMemcpyDeviceToHost);
  printf("PE %d: put_block of %zu ints from PE %d, %d wrong\n", me, N, (me + n - 1) % n, h_bad);
  cudaFree(bad);
  nvshmem_free(src);
  nvshmem_free(dst);
  nvshmem_finalize();
  return h_bad != 0;
}
