// Kernels that exercise the public device API (nvshmem.h) exactly as a user
// program would: compiled against the headers only, linked to the host library,
// launched from the Python test-suite and the perftest drivers through plain C
// entry points.  Every kernel writes what it observed into caller buffers; the
// host side compares with a CPU oracle.
#include <cuda_runtime.h>
#include <stdint.h>

#include "nvshmem.h"
#include "nvshmemx.h"

#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : 1)

// ------------------------------------------------------------------ RMA in every scope
// scope: 0 thread (thread 0 only), 1 warp (warp 0), 2 block.  nbi != 0 uses the non-blocking call + quiet.
__global__ void k_put(char* dst, const char* src, size_t bytes, int pe, int scope, int nbi) {
  if (scope == 0) {
    if (threadIdx.x == 0) {
      if (nbi) { nvshmem_putmem_nbi(dst, src, bytes, pe); nvshmem_quiet(); } else nvshmem_putmem(dst, src, bytes, pe);
    }
  } else if (scope == 1) {
    if (threadIdx.x < 32) {
      if (nbi) { nvshmemx_putmem_nbi_warp(dst, src, bytes, pe); nvshmemx_quiet_warp(); } else nvshmemx_putmem_warp(dst, src, bytes, pe);
    }
  } else {
    if (nbi) { nvshmemx_putmem_nbi_block(dst, src, bytes, pe); nvshmemx_quiet_block(); } else nvshmemx_putmem_block(dst, src, bytes, pe);
  }
}
__global__ void k_get(char* dst, const char* src, size_t bytes, int pe, int scope, int nbi) {
  if (scope == 0) {
    if (threadIdx.x == 0) {
      if (nbi) { nvshmem_getmem_nbi(dst, src, bytes, pe); nvshmem_quiet(); } else nvshmem_getmem(dst, src, bytes, pe);
    }
  } else if (scope == 1) {
    if (threadIdx.x < 32) {
      if (nbi) { nvshmemx_getmem_nbi_warp(dst, src, bytes, pe); nvshmemx_quiet_warp(); } else nvshmemx_getmem_warp(dst, src, bytes, pe);
    }
  } else {
    if (nbi) { nvshmemx_getmem_nbi_block(dst, src, bytes, pe); nvshmemx_quiet_block(); } else nvshmemx_getmem_block(dst, src, bytes, pe);
  }
}
// Typed calls: float put (block), int p/g, double iput/iget, bf16 put (warp).
__global__ void k_typed(float* fdst, const float* fsrc, int* idst, double* ddst, const double* dsrc, __nv_bfloat16* hdst, const __nv_bfloat16* hsrc, size_t n, int pe,
                        int* g_out) {
  nvshmemx_float_put_block(fdst, fsrc, n, pe);
  if (threadIdx.x < 32) nvshmemx_bfloat16_put_warp(hdst, hsrc, n, pe);
  if (threadIdx.x == 0) {
    nvshmem_int_p(idst, 1000 + nvshmem_my_pe(), pe);
    nvshmem_double_iput(ddst, dsrc, 2, 3, n / 4, pe);  // every 3rd source element to every 2nd slot
    nvshmem_quiet();
    g_out[0] = nvshmem_int_g(idst, pe);                 // reads back what was just written remotely
    g_out[1] = nvshmem_n_pes();
    g_out[2] = nvshmem_ptr(fdst, pe) != nullptr;
    g_out[3] = nvshmem_ptr(g_out, pe) == nullptr;       // g_out is not symmetric
  }
}

// ------------------------------------------------------------------ signals
__global__ void k_put_signal(char* dst, const char* src, size_t bytes, uint64_t* sig, uint64_t val, int op, int pe, int scope) {
  if (scope == 0) {
    if (threadIdx.x == 0) nvshmem_putmem_signal(dst, src, bytes, sig, val, op, pe);
  } else if (scope == 1) {
    if (threadIdx.x < 32) nvshmemx_putmem_signal_warp(dst, src, bytes, sig, val, op, pe);
  } else {
    nvshmemx_putmem_signal_block(dst, src, bytes, sig, val, op, pe);
  }
}
// Waits for the signal, then checksums the payload: the sum is only right if the data was visible.
__global__ void k_signal_wait_sum(const uint32_t* data, size_t nwords, uint64_t* sig, int cmp, uint64_t val, unsigned long long* out) {
  __shared__ unsigned long long partial;
  if (threadIdx.x == 0) {
    partial = 0;
    out[1] = nvshmem_signal_wait_until(sig, cmp, val);
  }
  __syncthreads();
  unsigned long long s = 0;
  for (size_t i = threadIdx.x; i < nwords; i += blockDim.x) s += data[i];
  atomicAdd(&partial, s);
  __syncthreads();
  if (threadIdx.x == 0) out[0] = partial;
}
// Ring: PE 0 starts a token; each PE waits for its signal, adds its rank to the token and forwards it.
__global__ void k_ring(uint64_t* token, uint64_t* sig, int rounds, uint64_t base) {
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes(), next = (me + 1) % n;
  for (int r = 0; r < rounds; ++r) {
    const uint64_t want = base + (uint64_t)r + 1;
    if (me != 0 || r > 0) nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, me == 0 ? want - 1 : want);
    uint64_t v = (me == 0 && r == 0) ? 0 : *(volatile uint64_t*)token;
    v += (uint64_t)me + 1;
    nvshmem_uint64_put_signal(token, &v, 1, sig, me == n - 1 ? want : want, NVSHMEM_SIGNAL_SET, next);
  }
  if (me == 0) nvshmem_signal_wait_until(sig, NVSHMEM_CMP_GE, base + (uint64_t)rounds);
}
// A wait that nothing satisfies: returns after the configured bound and reports the time-out.
__global__ void k_wait_never(uint64_t* sig, uint64_t val, int* out) {
  nvshmem_uint64_wait_until(sig, NVSHMEM_CMP_EQ, val);
  out[0] = (int)(nvshmemx_b200_device_error_bits() & BSHMEM_ERR_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ atomics
// Every thread of every CTA: fetch_add(1) on PE `pe`; old values must be a permutation of 0..N-1.
__global__ void k_amo_fetch_add(long long* target, int pe, long long* olds) {
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  olds[gid] = nvshmem_longlong_atomic_fetch_add(target, 1LL, pe);
}
__global__ void k_amo_mix(unsigned long long* t64, unsigned int* t32, float* tf, int pe, unsigned long long* out) {
  if (threadIdx.x != 0) return;
  const int me = nvshmem_my_pe();
  nvshmem_ulonglong_atomic_or(t64, 1ULL << me, pe);
  nvshmem_uint_atomic_add(t32, 3u, pe);
  nvshmem_uint_atomic_inc(t32, pe);
  out[0] = nvshmem_ulonglong_atomic_fetch(t64, pe);
  out[1] = nvshmem_uint_atomic_compare_swap(t32 + 1, 0u, 77u + me, pe);  // exactly one PE sees 0
  out[2] = (unsigned long long)__float_as_uint(nvshmem_float_atomic_swap(tf, 1.5f + me, pe));
  nvshmem_ulonglong_atomic_xor(t64 + 1, 0xffULL, pe);
  nvshmem_ulonglong_atomic_and(t64 + 2, ~(1ULL << me), pe);
}

// ------------------------------------------------------------------ barrier / sync at every scope
// Each round every PE writes (round, me) into slot `me` of the next PE, barriers, and checks the slot
// written by its predecessor.  errors[0] counts mismatches.
__global__ void k_barrier_rounds(long long* slots, int rounds, int scope, int* errors) {
  const int me = nvshmem_my_pe(), n = nvshmem_n_pes(), next = (me + 1) % n, prev = (me + n - 1) % n;
  for (int r = 1; r <= rounds; ++r) {
    if (threadIdx.x == 0) nvshmem_longlong_p(slots + me, (long long)r * 1000 + me, next);
    if (scope == 0) { if (threadIdx.x == 0) nvshmem_barrier_all(); __syncthreads(); }
    else if (scope == 1) { if (threadIdx.x < 32) nvshmemx_barrier_all_warp(); __syncthreads(); }
    else if (scope == 2) nvshmemx_barrier_all_block();
    else { if (threadIdx.x < 128) nvshmemx_barrier_all_warpgroup(); __syncthreads(); }
    if (threadIdx.x == 0 && *(volatile long long*)(slots + prev) != (long long)r * 1000 + prev) atomicAdd(errors, 1);
    // second barrier: nobody overwrites a slot before its reader has looked
    if (scope == 2) nvshmemx_sync_all_block();
    else { if (threadIdx.x == 0) nvshmem_sync_all(); __syncthreads(); }
  }
}

// ------------------------------------------------------------------ device-side collectives (block scope)
// kind: 0 float sum allreduce, 1 int max allreduce, 2 float sum reducescatter, 3 fcollect (int), 4 alltoall (int),
//       5 broadcast (int, root), 6 bf16 sum allreduce, 7 uint64 xor allreduce (warp scope), 8 int fcollect (thread scope)
__global__ void k_device_coll(int kind, int team, void* dst, const void* src, size_t n, int root, int* status) {
  int rc = 0;
  switch (kind) {
    case 0: rc = nvshmemx_float_sum_reduce_block(team, (float*)dst, (const float*)src, n); break;
    case 1: rc = nvshmemx_int_max_reduce_block(team, (int*)dst, (const int*)src, n); break;
    case 2: rc = nvshmemx_float_sum_reducescatter_block(team, (float*)dst, (const float*)src, n); break;
    case 3: rc = nvshmemx_int_fcollect_block(team, (int*)dst, (const int*)src, n); break;
    case 4: rc = nvshmemx_int_alltoall_block(team, (int*)dst, (const int*)src, n); break;
    case 5: rc = nvshmemx_int_broadcast_block(team, (int*)dst, (const int*)src, n, root); break;
    case 6: rc = nvshmemx_bfloat16_sum_reduce_block(team, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n); break;
    case 7: if (threadIdx.x < 32) rc = nvshmemx_uint64_xor_reduce_warp(team, (uint64_t*)dst, (const uint64_t*)src, n); break;
    case 8: if (threadIdx.x == 0) rc = nvshmem_int_fcollect(team, (int*)dst, (const int*)src, n); break;
  }
  if (threadIdx.x == 0) status[0] = rc;
}

// ------------------------------------------------------------------ tile API
// One CTA reduces a [rows x cols] tile located at (r0, c0) of a row-major [R x C] float tensor across the team.
__global__ void k_tile_allreduce(int team, float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int algo, int root) {
  using namespace nvshmemx;
  auto lay = make_layout(make_shape(rows, cols), make_stride(C, ConstInt<1>{}));
  Tensor<float, decltype(lay)> s(src + (size_t)r0 * C + c0, lay), d(dst + (size_t)r0 * C + c0, lay);
  auto start = make_shape(r0, c0);
  auto bound = make_shape(R, C);
  if (algo == 1) tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_ONE_SHOT_PULL_NBI>(team, s, d, start, bound, 0);
  else tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_TWO_SHOT_PUSH_NBI>(team, s, d, start, bound, root, 0);
  tile_collective_wait_block<NVLS_ONE_SHOT_PULL_NBI>(team, 0);
}
// The same with several CTAs at once: CTA b owns the tile whose first row is r0 + b * rows and synchronises on
// flag row b of the team, so the CTAs do not share a synchronisation epoch.
__global__ void k_tile_allreduce_multi(int team, float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int algo, int root) {
  using namespace nvshmemx;
  const int rb = r0 + (int)blockIdx.x * rows;
  auto lay = make_layout(make_shape(rows, cols), make_stride(C, ConstInt<1>{}));
  Tensor<float, decltype(lay)> s(src + (size_t)rb * C + c0, lay), d(dst + (size_t)rb * C + c0, lay);
  auto start = make_shape(rb, c0);
  auto bound = make_shape(R, C);
  if (algo == 1) tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_ONE_SHOT_PULL_NBI>(team, s, d, start, bound, blockIdx.x);
  else tile_sum_reduce_block<decltype(s), decltype(d), decltype(start), NVLS_TWO_SHOT_PUSH_NBI>(team, s, d, start, bound, root, blockIdx.x);
  tile_collective_wait_block<NVLS_ONE_SHOT_PULL_NBI>(team, blockIdx.x);
}
__global__ void k_tile_put_get(float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int pe, int get) {
  using namespace nvshmemx;
  auto lay = make_layout(make_shape(rows, cols), make_stride(C, 1));
  Tensor<float, decltype(lay)> s(src + (size_t)r0 * C + c0, lay), d(dst + (size_t)r0 * C + c0, lay);
  auto start = make_shape(r0, c0);
  auto bound = make_shape(R, C);
  if (get) tile_get_block<decltype(s), decltype(d), decltype(start), PEER_PULL_NBI>(s, d, start, bound, pe, 0);
  else tile_put_block<decltype(s), decltype(d), decltype(start), PEER_PUSH_NBI>(s, d, start, bound, pe, 0);
  nvshmemx_quiet_block();
}

// One call of each family of thin wrappers: queue-pair forms (the handle is accepted and ignored: load/store peers have
// no queue pairs), sized puts / gets, byte collectives at the three scopes.  `buf` is a symmetric int64 array of at
// least 64 + 8 * npes words, `sig` a symmetric signal word; results are checked on the host.
__global__ void k_api_wrappers(long long* buf, uint64_t* sig, int pe, int* status) {
  const nvshmemx_qp_handle_t qp = 0;
  nvshmemx_qp_handle_t qps[1] = {0};
  int rc = 0;
  if (threadIdx.x == 0) {
    nvshmemx_qp_longlong_p(buf + 0, 101LL, pe, qp);
    long long two[2] = {202LL, 203LL};
    nvshmemx_qp_longlong_put(buf + 1, two, 2, pe, qp);
    nvshmemx_qp_longlong_put_nbi(buf + 3, two, 2, pe, qp);
    nvshmemx_qp_quiet(0, qps, 1);
    nvshmemx_qp_fence(0, qps, 1);
    nvshmem_put64(buf + 5, two, 2, pe);
    nvshmem_put32(buf + 7, two, 2, pe);            // two 32-bit elements: the low word of two[0] and its high word
    nvshmem_put8(buf + 8, two, 8, pe);
    nvshmem_quiet();
  }
  __syncthreads();
  nvshmemx_qp_longlong_put_block(buf + 16, buf + 40, 8, pe, qp);   // whatever the source holds: compared with the source on the host
  nvshmemx_qp_quiet_block(0, qps, 1);
  if (threadIdx.x < 32) {
    nvshmemx_qp_longlong_put_signal_warp(buf + 24, buf + 40, 8, sig, 5ULL, NVSHMEM_SIGNAL_ADD, pe, qp);
    nvshmemx_qp_quiet_warp(0, qps, 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    nvshmemx_qp_signal_op(sig, 2ULL, NVSHMEM_SIGNAL_ADD, pe, qp);
    nvshmem_quiet();
  }
  // byte collectives: every PE contributes 8 bytes (its word 48), gathered into words 64 .. 64 + npes
  nvshmemx_barrier_all_block();
  rc |= nvshmemx_fcollectmem_block(NVSHMEM_TEAM_WORLD, buf + 64, buf + 48, 8);
  if (threadIdx.x < 32) rc |= nvshmemx_broadcastmem_warp(NVSHMEM_TEAM_WORLD, buf + 49, buf + 48, 8, 0);
  __syncthreads();
  if (threadIdx.x == 0) {
    rc |= nvshmem_alltoallmem(NVSHMEM_TEAM_WORLD, buf + 64 + nvshmem_n_pes(), buf + 64, 8);
    status[0] = rc;
    status[1] = (int)nvshmemx_qp_longlong_g(buf + 48, pe, qp);
  }
}

extern "C" {
// With lazy module loading the first launch of a kernel may have to wait for running kernels to
// finish.  Tests that start a waiting kernel before the kernel that satisfies it call this first.
int devtest_preload(void) {
  cudaFuncAttributes a;
  const void* fns[] = {(const void*)k_put, (const void*)k_get, (const void*)k_typed, (const void*)k_put_signal, (const void*)k_signal_wait_sum, (const void*)k_ring,
                       (const void*)k_wait_never, (const void*)k_amo_fetch_add, (const void*)k_amo_mix, (const void*)k_barrier_rounds, (const void*)k_device_coll,
                       (const void*)k_tile_allreduce, (const void*)k_tile_allreduce_multi, (const void*)k_tile_put_get, (const void*)k_api_wrappers};
  int bad = 0;
  for (const void* f : fns) bad |= cudaFuncGetAttributes(&a, f) != cudaSuccess;
  return bad;
}
int devtest_put(void* dst, const void* src, size_t bytes, int pe, int scope, int nbi, cudaStream_t s) {
  k_put<<<1, 256, 0, s>>>((char*)dst, (const char*)src, bytes, pe, scope, nbi);
  return LAUNCH_OK();
}
int devtest_get(void* dst, const void* src, size_t bytes, int pe, int scope, int nbi, cudaStream_t s) {
  k_get<<<1, 256, 0, s>>>((char*)dst, (const char*)src, bytes, pe, scope, nbi);
  return LAUNCH_OK();
}
int devtest_typed(float* fdst, const float* fsrc, int* idst, double* ddst, const double* dsrc, void* hdst, const void* hsrc, size_t n, int pe, int* g_out, cudaStream_t s) {
  k_typed<<<1, 128, 0, s>>>(fdst, fsrc, idst, ddst, dsrc, (__nv_bfloat16*)hdst, (const __nv_bfloat16*)hsrc, n, pe, g_out);
  return LAUNCH_OK();
}
int devtest_put_signal(void* dst, const void* src, size_t bytes, uint64_t* sig, uint64_t val, int op, int pe, int scope, cudaStream_t s) {
  k_put_signal<<<1, 256, 0, s>>>((char*)dst, (const char*)src, bytes, sig, val, op, pe, scope);
  return LAUNCH_OK();
}
int devtest_signal_wait_sum(const void* data, size_t nwords, uint64_t* sig, int cmp, uint64_t val, unsigned long long* out, cudaStream_t s) {
  k_signal_wait_sum<<<1, 256, 0, s>>>((const uint32_t*)data, nwords, sig, cmp, val, out);
  return LAUNCH_OK();
}
int devtest_ring(uint64_t* token, uint64_t* sig, int rounds, uint64_t base, cudaStream_t s) {
  k_ring<<<1, 1, 0, s>>>(token, sig, rounds, base);
  return LAUNCH_OK();
}
int devtest_wait_never(uint64_t* sig, uint64_t val, int* out, cudaStream_t s) {
  k_wait_never<<<1, 1, 0, s>>>(sig, val, out);
  return LAUNCH_OK();
}
int devtest_amo_fetch_add(long long* target, int pe, long long* olds, int ctas, int threads, cudaStream_t s) {
  k_amo_fetch_add<<<ctas, threads, 0, s>>>(target, pe, olds);
  return LAUNCH_OK();
}
int devtest_amo_mix(unsigned long long* t64, unsigned int* t32, float* tf, int pe, unsigned long long* out, cudaStream_t s) {
  k_amo_mix<<<1, 32, 0, s>>>(t64, t32, tf, pe, out);
  return LAUNCH_OK();
}
int devtest_barrier_rounds(long long* slots, int rounds, int scope, int* errors, cudaStream_t s) {
  k_barrier_rounds<<<1, 256, 0, s>>>(slots, rounds, scope, errors);
  return LAUNCH_OK();
}
int devtest_device_coll(int kind, int team, void* dst, const void* src, size_t n, int root, int* status, int threads, cudaStream_t s) {
  k_device_coll<<<1, threads, 0, s>>>(kind, team, dst, src, n, root, status);
  return LAUNCH_OK();
}
int devtest_tile_allreduce(int team, float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int algo, int root, cudaStream_t s) {
  k_tile_allreduce<<<1, 256, 0, s>>>(team, dst, src, R, C, r0, c0, rows, cols, algo, root);
  return LAUNCH_OK();
}
int devtest_tile_allreduce_multi(int team, float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int algo, int root, int ctas, cudaStream_t s) {
  if (ctas < 1 || ctas > BSHMEM_SYNC_SLOTS) return 1;
  k_tile_allreduce_multi<<<ctas, 256, 0, s>>>(team, dst, src, R, C, r0, c0, rows, cols, algo, root);
  return LAUNCH_OK();
}
int devtest_api_wrappers(long long* buf, uint64_t* sig, int pe, int* status, cudaStream_t s) {
  k_api_wrappers<<<1, 128, 0, s>>>(buf, sig, pe, status);
  return LAUNCH_OK();
}
int devtest_tile_put_get(float* dst, float* src, int R, int C, int r0, int c0, int rows, int cols, int pe, int get, cudaStream_t s) {
  k_tile_put_get<<<1, 256, 0, s>>>(dst, src, R, C, r0, c0, rows, cols, pe, get);
  return LAUNCH_OK();
}
}
