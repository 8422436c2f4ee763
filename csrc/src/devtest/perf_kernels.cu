// Timing kernels of the perftest drivers (put/get bandwidth, ping-pong latency, atomics, barrier and
// device-collective latency), written against the public device API.  Each kernel performs `iters`
// operations so that one launch amortises launch overhead; the host times the launch with CUDA events
// (reference method: perftest/device/pt-to-pt/shmem_put_bw.cu, shmem_put_signal_ping_pong_latency.cu,
//  perftest/common/atomic_bw_common.h, perftest/device/coll/*_latency.cu).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "nvshmem.h"
#include "nvshmemx.h"

// Inter-CTA barrier inside one launch (all CTAs co-resident: grids here never exceed the SM count).
__device__ __forceinline__ void cta_rendezvous(unsigned* counter, unsigned target) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    const unsigned long long start = bshmem::global_timer_ns();
    while (*(volatile unsigned*)counter < target) {
      if (bshmem::global_timer_ns() - start > 5000000000ull) break;  // bounded
    }
  }
  __syncthreads();
}

// scope: 0 thread (each thread moves its own piece), 1 warp, 2 block.  `dir` 0 = put, 1 = get.
__global__ void __launch_bounds__(1024) k_bw(char* sym, char* local, size_t bytes, int pe, int iters, int scope, int dir, unsigned* counter) {
  const size_t per_cta = (bytes / gridDim.x) & ~(size_t)15;
  char* s = sym + (size_t)blockIdx.x * per_cta;
  char* l = local + (size_t)blockIdx.x * per_cta;
  for (int it = 0; it < iters; ++it) {
    if (scope == 2) {
      if (dir == 0) nvshmemx_putmem_nbi_block(s, l, per_cta, pe);
      else nvshmemx_getmem_nbi_block(l, s, per_cta, pe);
    } else if (scope == 1) {
      const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
      const size_t per_w = (per_cta / nw) & ~(size_t)15;
      if (dir == 0) nvshmemx_putmem_nbi_warp(s + w * per_w, l + w * per_w, per_w, pe);
      else nvshmemx_getmem_nbi_warp(l + w * per_w, s + w * per_w, per_w, pe);
    } else {
      const size_t per_t = (per_cta / blockDim.x) & ~(size_t)15;
      if (per_t) {
        if (dir == 0) nvshmem_putmem_nbi(s + threadIdx.x * per_t, l + threadIdx.x * per_t, per_t, pe);
        else nvshmem_getmem_nbi(l + threadIdx.x * per_t, s + threadIdx.x * per_t, per_t, pe);
      }
    }
    cta_rendezvous(counter, (unsigned)(it + 1) * gridDim.x);
  }
  nvshmemx_quiet_block();
}

// Store bandwidth: plain stores through the peer's mapped address (nvshmem_ptr), two 8-byte elements in flight per
// thread, the way a kernel writes a peer buffer without any library call (reference: perftest/device/pt-to-pt/shmem_st_bw.cu).
__global__ void __launch_bounds__(1024) k_st_bw(double* sym, const double* local, size_t len, int pe, int iters, unsigned* counter) {
  double* remote = (double*)nvshmem_ptr(sym, pe);
  const size_t threads = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int it = 0; it < iters; ++it) {
    if (remote) {
      size_t j = tid;
      for (; j + threads < len; j += 2 * threads) {
        const double a = local[j], b = local[j + threads];
        remote[j] = a;
        remote[j + threads] = b;
      }
      if (j < len) remote[j] = local[j];
    }
    cta_rendezvous(counter, (unsigned)(it + 1) * gridDim.x);
  }
  nvshmemx_quiet_block();
}

// Small-message rate: every thread issues `iters` single-element puts (p) or gets (g).
__global__ void __launch_bounds__(1024) k_pg_rate(unsigned long long* sym, int pe, int iters, int dir, unsigned long long* sink) {
  unsigned long long acc = 0;
  unsigned long long* slot = sym + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int it = 0; it < iters; ++it) {
    if (dir == 0) nvshmem_ulonglong_p(slot, (unsigned long long)it, pe);
    else acc += nvshmem_ulonglong_g(slot, pe);
  }
  nvshmem_quiet();
  if (acc == 0xdeadbeefULL) *sink = acc;
}

// Blocking latency of one operation issued by a single thread / warp / block: `iters` put + quiet round trips.
__global__ void __launch_bounds__(1024) k_put_latency(char* sym, char* local, size_t bytes, int pe, int iters, int scope) {
  for (int it = 0; it < iters; ++it) {
    if (scope == 2) { nvshmemx_putmem_block(sym, local, bytes, pe); nvshmemx_quiet_block(); }
    else if (scope == 1) { if (threadIdx.x < 32) { nvshmemx_putmem_warp(sym, local, bytes, pe); nvshmemx_quiet_warp(); } }
    else if (threadIdx.x == 0) { nvshmem_putmem(sym, local, bytes, pe); nvshmem_quiet(); }
  }
}
// Each get starts where the previous one's data says (the driver zeroes the source buffer, so always offset 0):
// the chain makes consecutive gets dependent, so the time per iteration is a latency, not a rate.
__global__ void __launch_bounds__(1024) k_get_latency(char* sym, char* local, size_t bytes, int pe, int iters, int scope) {
  __shared__ size_t off;
  if (threadIdx.x == 0) off = 0;
  __syncthreads();
  for (int it = 0; it < iters; ++it) {
    if (scope == 2) nvshmemx_getmem_block(local, sym + off, bytes, pe);
    else if (scope == 1) { if (threadIdx.x < 32) nvshmemx_getmem_warp(local, sym + off, bytes, pe); }
    else if (threadIdx.x == 0) nvshmem_getmem(local, sym + off, bytes, pe);
    __syncthreads();
    if (threadIdx.x == 0) off = (size_t)(*(volatile unsigned char*)local);  // data-dependent; the data is zero
    __syncthreads();
  }
}

// Ping-pong between PE 0 and PE 1 with put_signal: half the round trip is the one-way latency.
__global__ void __launch_bounds__(1024) k_pingpong(char* data, char* local, size_t bytes, uint64_t* sig, int iters, uint64_t base, int scope) {
  const int me = nvshmem_my_pe(), peer = 1 - me;
  if (me > 1) return;
  for (int it = 1; it <= iters; ++it) {
    const uint64_t v = base + (uint64_t)it;
    if (me == 0) {
      if (scope == 2) nvshmemx_putmem_signal_block(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer);
      else if (scope == 1) { if (threadIdx.x < 32) nvshmemx_putmem_signal_warp(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer); }
      else if (threadIdx.x == 0) nvshmem_putmem_signal(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer);
      if (threadIdx.x == 0) nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, v);
      __syncthreads();
    } else {
      if (threadIdx.x == 0) nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, v);
      __syncthreads();
      if (scope == 2) nvshmemx_putmem_signal_block(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer);
      else if (scope == 1) { if (threadIdx.x < 32) nvshmemx_putmem_signal_warp(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer); }
      else if (threadIdx.x == 0) nvshmem_putmem_signal(data, local, bytes, sig, v, NVSHMEM_SIGNAL_SET, peer);
    }
  }
}
// Signal-only ping-pong (no payload).
__global__ void __launch_bounds__(1024) k_signal_pingpong(uint64_t* sig, int iters, uint64_t base) {
  const int me = nvshmem_my_pe(), peer = 1 - me;
  if (me > 1 || threadIdx.x) return;
  for (int it = 1; it <= iters; ++it) {
    const uint64_t v = base + (uint64_t)it;
    if (me == 0) {
      nvshmemx_signal_op(sig, v, NVSHMEM_SIGNAL_SET, peer);
      nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, v);
    } else {
      nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, v);
      nvshmemx_signal_op(sig, v, NVSHMEM_SIGNAL_SET, peer);
    }
  }
}

// Atomic throughput: every thread performs `iters` operations on its own 64-bit word of PE `pe`, or all on one word
// when `contend`.  kind: 0 fetch_add, 1 add, 2 compare_swap, 3 swap, 4 fetch_or, 5 inc, 6 fetch_inc, 7 and, 8 fetch_and,
// 9 or, 10 xor, 11 fetch_xor, 12 set (the thirteen operations of the reference's atomic bandwidth test).
__global__ void __launch_bounds__(1024) k_atomic_rate(long long* sym, int pe, int iters, int kind, int contend, long long* sink) {
  long long* t = contend ? sym : sym + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint64_t* u = (uint64_t*)t;
  long long acc = 0;
  for (int it = 0; it < iters; ++it) {
    switch (kind) {
      case 0: acc += nvshmem_longlong_atomic_fetch_add(t, 1LL, pe); break;
      case 1: nvshmem_longlong_atomic_add(t, 1LL, pe); break;
      case 2: acc += nvshmem_longlong_atomic_compare_swap(t, (long long)it, (long long)it + 1, pe); break;
      case 3: acc += nvshmem_longlong_atomic_swap(t, (long long)it, pe); break;
      case 4: acc += (long long)nvshmem_uint64_atomic_fetch_or(u, 1ULL << (it & 63), pe); break;
      case 5: nvshmem_longlong_atomic_inc(t, pe); break;
      case 6: acc += nvshmem_longlong_atomic_fetch_inc(t, pe); break;
      case 7: nvshmem_uint64_atomic_and(u, ~(1ULL << (it & 63)), pe); break;
      case 8: acc += (long long)nvshmem_uint64_atomic_fetch_and(u, ~(1ULL << (it & 63)), pe); break;
      case 9: nvshmem_uint64_atomic_or(u, 1ULL << (it & 63), pe); break;
      case 10: nvshmem_uint64_atomic_xor(u, 1ULL, pe); break;
      case 11: acc += (long long)nvshmem_uint64_atomic_fetch_xor(u, 1ULL, pe); break;
      default: nvshmem_longlong_atomic_set(t, (long long)it + 1, pe); break;
    }
  }
  nvshmem_quiet();
  if (acc == 0x7fffffffffffffffLL) *sink = acc;
}
// Latency of a dependent chain of fetching atomics by one thread.
__global__ void __launch_bounds__(1024) k_atomic_latency(long long* sym, int pe, int iters, long long* sink) {
  if (threadIdx.x || blockIdx.x) return;
  long long v = 0;
  for (int it = 0; it < iters; ++it) v = nvshmem_longlong_atomic_fetch_add(sym, v & 1, pe);
  *sink = v;
}

// Barrier / sync latency at each scope.
__global__ void __launch_bounds__(1024) k_barrier_latency(int iters, int scope, int sync_only) {
  for (int it = 0; it < iters; ++it) {
    if (scope == 2) { if (sync_only) nvshmemx_sync_all_block(); else nvshmemx_barrier_all_block(); }
    else if (scope == 1) { if (threadIdx.x < 32) { if (sync_only) nvshmemx_sync_all_warp(); else nvshmemx_barrier_all_warp(); } }
    else if (threadIdx.x == 0) { if (sync_only) nvshmem_sync_all(); else nvshmem_barrier_all(); }
  }
}

// Device-initiated collectives, `iters` back to back (block scope).  kind as in the test kernels:
// 0 float sum allreduce, 2 float sum reducescatter, 3 int fcollect, 4 int alltoall, 5 int broadcast, 6 bf16 sum allreduce.
__global__ void __launch_bounds__(1024) k_coll_latency(int kind, void* dst, const void* src, size_t n, int iters) {
  for (int it = 0; it < iters; ++it) {
    switch (kind) {
      case 0: nvshmemx_float_sum_reduce_block(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
      case 2: nvshmemx_float_sum_reducescatter_block(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
      case 3: nvshmemx_int_fcollect_block(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
      case 4: nvshmemx_int_alltoall_block(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
      case 5: nvshmemx_int_broadcast_block(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n, 0); break;
      default: nvshmemx_bfloat16_sum_reduce_block(NVSHMEM_TEAM_WORLD, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n); break;
    }
  }
}

// The same collectives issued by one thread (scope 0) or one warp (scope 1) of the CTA, and the (value, index)
// maximum (kind 7: double2 max-location at block scope; reference: perftest/device/coll/redmaxloc_latency.cu).
__global__ void __launch_bounds__(1024) k_coll_latency_scoped(int kind, void* dst, const void* src, size_t n, int iters, int scope) {
  if (kind == 7) {
    for (int it = 0; it < iters; ++it) nvshmemx_double2_maxloc_reduce_block(NVSHMEM_TEAM_WORLD, (double2*)dst, (const double2*)src, 1);
    return;
  }
  if (scope == 0 && threadIdx.x != 0) return;
  if (scope == 1 && threadIdx.x >= 32) return;
  for (int it = 0; it < iters; ++it) {
    if (scope == 0) {
      switch (kind) {
        case 0: nvshmem_float_sum_reduce(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
        case 2: nvshmem_float_sum_reducescatter(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
        case 3: nvshmem_int_fcollect(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
        case 4: nvshmem_int_alltoall(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
        case 5: nvshmem_int_broadcast(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n, 0); break;
        default: nvshmem_bfloat16_sum_reduce(NVSHMEM_TEAM_WORLD, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n); break;
      }
    } else {
      switch (kind) {
        case 0: nvshmemx_float_sum_reduce_warp(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
        case 2: nvshmemx_float_sum_reducescatter_warp(NVSHMEM_TEAM_WORLD, (float*)dst, (const float*)src, n); break;
        case 3: nvshmemx_int_fcollect_warp(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
        case 4: nvshmemx_int_alltoall_warp(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n); break;
        case 5: nvshmemx_int_broadcast_warp(NVSHMEM_TEAM_WORLD, (int*)dst, (const int*)src, n, 0); break;
        default: nvshmemx_bfloat16_sum_reduce_warp(NVSHMEM_TEAM_WORLD, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n); break;
      }
    }
  }
}

#define OK() (cudaGetLastError() == cudaSuccess ? 0 : 1)
// Tile all-reduce / all-gather latency at block scope: `iters` collectives on a rows x cols fp32 tile of a
// row-major matrix with `ld` columns (reference: perftest/device/tile/tile_allreduce_latency.cu, tile_allgather_latency.cu).
__global__ void __launch_bounds__(1024) k_tile_latency(int kind, float* dst, float* src, int rows, int cols, int ld, int iters) {
  using namespace nvshmemx;
  auto lay = make_layout(make_shape(rows, cols), make_stride(ld, ConstInt<1>{}));
  // all-gather: every PE's tile lands in its own slot of the destination
  Tensor<float, decltype(lay)> s(src, lay), d(kind == 2 ? dst + (size_t)nvshmem_my_pe() * rows * ld : dst, lay);
  auto start = make_shape(0, 0);
  auto bound = make_shape(rows, ld);
  for (int i = 0; i < iters; ++i) {
    if (kind == 0) tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_ONE_SHOT_PULL_NBI>(NVSHMEM_TEAM_WORLD, s, d, start, bound, 0);
    else if (kind == 1) tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_TWO_SHOT_PUSH_NBI>(NVSHMEM_TEAM_WORLD, s, d, start, bound, 0, 0);
    else tile_allgather_block<decltype(s), decltype(d), decltype(start), NVLS_ONE_SHOT_PUSH_NBI>(NVSHMEM_TEAM_WORLD, s, d, start, bound, 0);
    tile_collective_wait_block<NVLS_ONE_SHOT_PUSH_NBI>(NVSHMEM_TEAM_WORLD, 0);
  }
}

extern "C" {
int perf_onstream_loop_algo(int kind, void* dst, const void* src, size_t bytes, int pe, int iters, int algo, int dtype, cudaStream_t s);
int perf_preload(void) {
  cudaFuncAttributes a;
  const void* fns[] = {(const void*)k_bw, (const void*)k_pg_rate, (const void*)k_put_latency, (const void*)k_get_latency, (const void*)k_pingpong,
                       (const void*)k_signal_pingpong, (const void*)k_atomic_rate, (const void*)k_atomic_latency, (const void*)k_barrier_latency,
                       (const void*)k_coll_latency, (const void*)k_tile_latency, (const void*)k_st_bw, (const void*)k_coll_latency_scoped};
  int bad = 0, i = 0;
  for (const void* f : fns) {
    cudaError_t e = cudaFuncGetAttributes(&a, f);
    if (e != cudaSuccess) {
      fprintf(stderr, "perf_preload: kernel %d: %s\n", i, cudaGetErrorString(e));
      bad = 1;
    }
    ++i;
  }
  return bad;
}
int perf_bw(void* sym, void* local, size_t bytes, int pe, int iters, int scope, int dir, int ctas, int threads, unsigned* counter, cudaStream_t s) {
  cudaMemsetAsync(counter, 0, sizeof(unsigned), s);
  k_bw<<<ctas, threads, 0, s>>>((char*)sym, (char*)local, bytes, pe, iters, scope, dir, counter);
  return OK();
}
int perf_pg_rate(void* sym, int pe, int iters, int dir, int ctas, int threads, void* sink, cudaStream_t s) {
  k_pg_rate<<<ctas, threads, 0, s>>>((unsigned long long*)sym, pe, iters, dir, (unsigned long long*)sink);
  return OK();
}
int perf_put_latency(void* sym, void* local, size_t bytes, int pe, int iters, int scope, int threads, cudaStream_t s) {
  k_put_latency<<<1, threads, 0, s>>>((char*)sym, (char*)local, bytes, pe, iters, scope);
  return OK();
}
int perf_get_latency(void* sym, void* local, size_t bytes, int pe, int iters, int scope, int threads, cudaStream_t s) {
  k_get_latency<<<1, threads, 0, s>>>((char*)sym, (char*)local, bytes, pe, iters, scope);
  return OK();
}
int perf_pingpong(void* data, void* local, size_t bytes, uint64_t* sig, int iters, uint64_t base, int scope, int threads, cudaStream_t s) {
  k_pingpong<<<1, threads, 0, s>>>((char*)data, (char*)local, bytes, sig, iters, base, scope);
  return OK();
}
int perf_signal_pingpong(uint64_t* sig, int iters, uint64_t base, cudaStream_t s) {
  k_signal_pingpong<<<1, 32, 0, s>>>(sig, iters, base);
  return OK();
}
int perf_atomic_rate(void* sym, int pe, int iters, int kind, int contend, int ctas, int threads, void* sink, cudaStream_t s) {
  k_atomic_rate<<<ctas, threads, 0, s>>>((long long*)sym, pe, iters, kind, contend, (long long*)sink);
  return OK();
}
int perf_atomic_latency(void* sym, int pe, int iters, void* sink, cudaStream_t s) {
  k_atomic_latency<<<1, 32, 0, s>>>((long long*)sym, pe, iters, (long long*)sink);
  return OK();
}
int perf_barrier_latency(int iters, int scope, int sync_only, int threads, cudaStream_t s) {
  k_barrier_latency<<<1, threads, 0, s>>>(iters, scope, sync_only);
  return OK();
}
int perf_coll_latency(int kind, void* dst, const void* src, size_t n, int iters, int threads, cudaStream_t s) {
  k_coll_latency<<<1, threads, 0, s>>>(kind, dst, src, n, iters);
  return OK();
}
// scope: 0 thread, 1 warp, 2 block; kind 7 = double2 max-location (block scope).
int perf_coll_latency_scoped(int kind, void* dst, const void* src, size_t n, int iters, int scope, int threads, cudaStream_t s) {
  if (scope == 2 && kind != 7) return perf_coll_latency(kind, dst, src, n, iters, threads, s);
  k_coll_latency_scoped<<<1, threads, 0, s>>>(kind, dst, src, n, iters, scope);
  return OK();
}
int perf_st_bw(void* sym, const void* local, size_t bytes, int pe, int iters, int ctas, int threads, unsigned* counter, cudaStream_t s) {
  cudaMemsetAsync(counter, 0, sizeof(unsigned), s);
  k_st_bw<<<ctas, threads, 0, s>>>((double*)sym, (const double*)local, bytes / 8, pe, iters, counter);
  return OK();
}
int perf_tile_latency(int kind, float* dst, float* src, int rows, int cols, int ld, int iters, int threads, cudaStream_t s) {
  k_tile_latency<<<1, threads, 0, s>>>(kind, dst, src, rows, cols, ld, iters);
  return OK();
}
// Issues `iters` on-stream calls of one kind back to back from C, the way the reference's host perftests do
// (no interpreter between the launches).  kind: 0 float sum all-reduce, 1 float sum reduce-scatter, 2 fcollect,
// 3 alltoall, 4 broadcast from PE 0, 5 barrier_all, 6 sync_all, 7 putmem to `pe`, 8 getmem from `pe`.
// `bytes` is the whole buffer per PE (block size = bytes / npes where the call works on blocks).
int perf_onstream_loop(int kind, void* dst, const void* src, size_t bytes, int pe, int iters, cudaStream_t s) {
  return perf_onstream_loop_algo(kind, dst, src, bytes, pe, iters, 0, 10 /* float */, s);
}
// The same with a forced algorithm (the numbering of the library's algorithm enums; 0 = automatic) and element type
// of the reductions (the library's type codes: 9 bfloat16, 10 float, 8 half, 4 int32 ...).
int perf_onstream_loop_algo(int kind, void* dst, const void* src, size_t bytes, int pe, int iters, int algo, int dtype, cudaStream_t s) {
  const int n = nvshmem_n_pes();
  const size_t es = dtype == 8 || dtype == 9 || dtype == 2 || dtype == 3 ? 2 : dtype == 11 || dtype == 6 || dtype == 7 ? 8 : dtype <= 1 ? 1 : 4;
  int st = 0;
  for (int i = 0; i < iters && !st; ++i) {
    switch (kind) {
      case 0: st = nvshmemx_b200_reduce_on_stream(NVSHMEM_TEAM_WORLD, dst, src, bytes / es, dtype, 5 /* sum */, algo, s); break;
      case 1: st = nvshmemx_b200_reducescatter_on_stream(NVSHMEM_TEAM_WORLD, dst, src, bytes / es / n, dtype, 5, algo, s); break;
      case 2: st = nvshmemx_b200_fcollect_on_stream(NVSHMEM_TEAM_WORLD, dst, src, bytes / n, algo, s); break;
      case 3: st = nvshmemx_alltoallmem_on_stream(NVSHMEM_TEAM_WORLD, dst, src, bytes / n, s); break;
      case 4: st = nvshmemx_b200_broadcast_on_stream(NVSHMEM_TEAM_WORLD, dst, src, bytes, 0, algo, s); break;
      case 5: nvshmemx_barrier_all_on_stream(s); break;
      case 6: nvshmemx_sync_all_on_stream(s); break;
      case 7: nvshmemx_putmem_on_stream(dst, src, bytes, pe, s); break;
      case 8: nvshmemx_getmem_on_stream(dst, src, bytes, pe, s); break;
      default: return 1;
    }
  }
  return st;
}
}
