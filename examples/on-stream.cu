// Stream-ordered communication: a kernel produces data, the library's on-stream calls move and reduce
// it, a second kernel consumes it; the host only enqueues.
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/on-stream
// (counterpart of the reference's examples/on-stream.cu)
#include <cuda_runtime.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

constexpr int N = 1 << 16;

__global__ void fill(float* x, float v) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) x[i] = v;
}
__global__ void check(const float* x, float want, int* bad) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x)
    if (x[i] != want) atomicAdd(bad, 1);
}

int main() {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  cudaStream_t s;
  cudaStreamCreate(&s);
  float* src = (float*)nvshmem_malloc(N * sizeof(float));
  float* dst = (float*)nvshmem_malloc(N * sizeof(float));
  int* bad;
  cudaMalloc(&bad, sizeof(int));
  cudaMemsetAsync(bad, 0, sizeof(int), s);
  fill<<<64, 256, 0, s>>>(src, (float)(me + 1));
  nvshmemx_float_sum_reduce_on_stream(NVSHMEM_TEAM_WORLD, dst, src, N, s);  // orders itself after `fill`
  check<<<64, 256, 0, s>>>(dst, (float)(n * (n + 1) / 2), bad);
  // the neighbour's source buffer, fetched on the stream
  nvshmemx_float_get_on_stream(dst, src, N, (me + 1) % n, s);
  check<<<64, 256, 0, s>>>(dst, (float)((me + 1) % n + 1), bad);
  nvshmemx_barrier_all_on_stream(s);
  int h_bad = -1;
  cudaMemcpyAsync(&h_bad, bad, sizeof(int), cudaMemcpyDeviceToHost, s);
  cudaStreamSynchronize(s);
  printf("PE %d: on-stream reduce + get, %d wrong elements\n", me, h_bad);
  cudaFree(bad);
  nvshmem_free(src);
  nvshmem_free(dst);
  nvshmem_finalize();
  return h_bad != 0;
}
