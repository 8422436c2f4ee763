// Chunked ring all-reduce written with put_signal and signal_wait_until: a reduce phase (each chunk
// travels the ring collecting sums) followed by a broadcast phase.  Every CTA owns one slice of the
// buffer and one pair of signals, so CTAs never wait on each other.
//   python -m nvshmem_b200.launch -n 4 -- examples/bin/ring-reduce
// Self-validating: with input element = index on every PE the result is index * npes.
// (counterpart of the reference's examples/ring-reduce.cu)
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include "nvshmem.h"
#include "nvshmemx.h"

constexpr int CTAS = 32, THREADS = 512;
constexpr size_t CHUNK = 64 * 1024;  // ints per chunk

// dst, src: symmetric, `nreduce` ints.  signals: symmetric, 2 per CTA (reduce phase, broadcast phase).
__global__ void ring_allreduce(int* dst, const int* src, size_t nreduce, uint64_t* signals) {
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  const int peer = (me + 1) % n;
  const size_t per_cta = nreduce / gridDim.x;
  int* d = dst + blockIdx.x * per_cta;
  const int* s = src + blockIdx.x * per_cta;
  uint64_t* sig_reduce = signals + 2 * blockIdx.x;
  uint64_t* sig_bcast = sig_reduce + 1;
  const size_t chunks = per_cta / CHUNK;
  if (n == 1) {  // nothing to exchange
    for (size_t i = threadIdx.x; i < per_cta; i += blockDim.x) d[i] = s[i];
    return;
  }
  // Reduce phase: PE 0 starts each chunk; PE i adds its part and forwards; PE n-1 ends up with the sum.
  for (size_t c = 0; c < chunks; ++c) {
    int* dc = d + c * CHUNK;
    const int* sc = s + c * CHUNK;
    if (me != 0) {
      if (threadIdx.x == 0) nvshmem_signal_wait_until(sig_reduce, NVSHMEM_CMP_GE, c + 1);
      __syncthreads();
      for (size_t i = threadIdx.x; i < CHUNK; i += blockDim.x) dc[i] += sc[i];
      __syncthreads();
    }
    if (me != n - 1) nvshmemx_int_put_signal_nbi_block(dc, me == 0 ? sc : dc, CHUNK, sig_reduce, 1, NVSHMEM_SIGNAL_ADD, peer);
  }
  // Broadcast phase: PE n-1 holds the sums; they go round once more (n-1 -> 0 -> 1 ... -> n-2).
  for (size_t c = 0; c < chunks; ++c) {
    int* dc = d + c * CHUNK;
    if (me != n - 1) {
      if (threadIdx.x == 0) nvshmem_signal_wait_until(sig_bcast, NVSHMEM_CMP_GE, c + 1);
      __syncthreads();
    }
    if (peer != n - 1) nvshmemx_int_put_signal_nbi_block(dc, dc, CHUNK, sig_bcast, 1, NVSHMEM_SIGNAL_ADD, peer);
  }
  // All my puts are complete before the kernel ends, so that the host-side barrier closes the operation.
  nvshmem_quiet();
}

int main(int argc, char** argv) {
  nvshmem_init();
  cudaSetDevice(nvshmem_team_my_pe(NVSHMEMX_TEAM_NODE));
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes();
  size_t mbytes = argc > 1 ? strtoul(argv[1], nullptr, 10) : 32;
  size_t nreduce = mbytes * 1024 * 1024 / sizeof(int);
  nreduce -= nreduce % (CTAS * CHUNK);
  int* src = (int*)nvshmem_malloc(nreduce * sizeof(int));
  int* dst = (int*)nvshmem_calloc(nreduce, sizeof(int));
  uint64_t* signals = (uint64_t*)nvshmem_calloc(2 * CTAS, sizeof(uint64_t));
  int* host = (int*)malloc(nreduce * sizeof(int));
  for (size_t i = 0; i < nreduce; ++i) host[i] = (int)i;
  cudaMemcpy(src, host, nreduce * sizeof(int), cudaMemcpyHostToDevice);
  nvshmem_barrier_all();
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  void* args[] = {&dst, &src, &nreduce, &signals};
  cudaEventRecord(t0, 0);
  int st = nvshmemx_collective_launch((const void*)ring_allreduce, dim3(CTAS), dim3(THREADS), args, 0, 0);
  cudaEventRecord(t1, 0);
  cudaDeviceSynchronize();
  nvshmem_barrier_all();
  float ms = 0;
  cudaEventElapsedTime(&ms, t0, t1);
  cudaMemcpy(host, dst, nreduce * sizeof(int), cudaMemcpyDeviceToHost);
  size_t bad = 0;
  for (size_t i = 0; i < nreduce; ++i) bad += host[i] != (int)i * n;
  printf("PE %d: ring all-reduce of %zu MB in %.3f ms, launch status %d, %zu wrong\n", me, nreduce * sizeof(int) >> 20, ms, st, bad);
  free(host);
  nvshmem_free(src);
  nvshmem_free(dst);
  nvshmem_free(signals);
  nvshmem_finalize();
  return bad != 0 || st != 0;
}
