// On-stream collectives: kernel instantiations of the device algorithms and
// their launchers.  A launch uses one CTA for small messages and several for
// large ones; CTA c reduces / moves its own element slice and synchronises with
// CTA c of every other PE through row c of the team's barrier flags, so no team
// is cloned and nothing is created during CUDA-graph capture.  The grid never
// exceeds BSHMEM_SYNC_SLOTS-1 CTAs, far below the SM count, so that the CTAs of
// all PEs are co-resident.
// (reference behaviour: src/include/internal/non_abi/nvshmemi_h_to_d_coll_defs.cuh,
//  src/host/stream/coll/**: thresholds 256 KiB reduce, 1 MiB fcollect / reducescatter)
#include <algorithm>

#include "../../include/bshmem/coll.cuh"
#include "../../include/bshmem/types.h"
#include "../state/runtime.h"
#include "../util/env.h"
#include "../util/log.h"
#include "../util/nvtx.h"
#include "coll_host.h"

namespace bshmem {

static constexpr int kHostSlot = BSHMEM_SYNC_SLOTS - 1;  // barrier flags of host-launched barriers

// ------------------------------------------------------------------ kernels
template <class T, int OP>
__global__ void reduce_kernel(int team, T* dst, const T* src, size_t n, int algo) {
  const bshmemi_team_t* t = team_ptr(team);
  size_t lo, hi;
  split_range<T>(n, gridDim.x, blockIdx.x, &lo, &hi);
  allreduce_range<T, OP, SCOPE_BLOCK>(t, dst, src, lo, hi, blockIdx.x, algo);
}
template <class T, int OP>
__global__ void reducescatter_kernel(int team, T* dst, const T* src, size_t nreduce, int algo) {
  const bshmemi_team_t* t = team_ptr(team);
  size_t lo, hi;
  split_range<T>(nreduce, gridDim.x, blockIdx.x, &lo, &hi);
  reducescatter_range<T, OP, SCOPE_BLOCK>(t, dst, src, nreduce, lo, hi, blockIdx.x, algo);
}
__global__ void fcollect_kernel(int team, void* dst, const void* src, size_t block_bytes, int algo) {
  const bshmemi_team_t* t = team_ptr(team);
  size_t lo, hi;
  split_range<uint8_t>(block_bytes, gridDim.x, blockIdx.x, &lo, &hi);
  fcollect_bytes<SCOPE_BLOCK>(t, dst, src, block_bytes, lo, hi, blockIdx.x, gridDim.x > 1 && algo == FC_AUTO ? FC_AUTO : algo);
}
__global__ void alltoall_kernel(int team, void* dst, const void* src, size_t block_bytes) {
  const bshmemi_team_t* t = team_ptr(team);
  size_t lo, hi;
  split_range<uint8_t>(block_bytes, gridDim.x, blockIdx.x, &lo, &hi);
  alltoall_bytes<SCOPE_BLOCK>(t, dst, src, block_bytes, lo, hi, blockIdx.x);
}
__global__ void broadcast_kernel(int team, void* dst, const void* src, size_t bytes, int root, int algo) {
  const bshmemi_team_t* t = team_ptr(team);
  size_t lo, hi;
  split_range<uint8_t>(bytes, gridDim.x, blockIdx.x, &lo, &hi);
  broadcast_bytes<SCOPE_BLOCK>(t, dst, src, lo, hi, root, blockIdx.x, algo);
}
__global__ void barrier_kernel(int team, int slot, int with_quiet) {
  const bshmemi_team_t* t = team_ptr(team);
  if (with_quiet) team_barrier<SCOPE_BLOCK>(t, slot);
  else team_sync<SCOPE_BLOCK>(t, slot);
}
__global__ void maxloc_kernel(int team, double2* dst, const double2* src) { maxloc_double2<SCOPE_BLOCK>(team, dst, src); }

// single-thread helpers of the on-stream point-to-point API
__global__ void wait_until_kernel(const uint64_t* ivar, int cmp, uint64_t value, int width) {
  if (width == 8) wait_until<uint64_t>(ivar, cmp, value);
  else if (width == 4) wait_until<uint32_t>((const uint32_t*)ivar, cmp, (uint32_t)value);
  else wait_until<uint16_t>((const uint16_t*)ivar, cmp, (uint16_t)value);
}
__global__ void wait_until_signed_kernel(const int64_t* ivar, int cmp, int64_t value, int width) {
  if (width == 8) wait_until<int64_t>(ivar, cmp, value);
  else if (width == 4) wait_until<int32_t>((const int32_t*)ivar, cmp, (int32_t)value);
  else wait_until<int16_t>((const int16_t*)ivar, cmp, (int16_t)value);
}
__global__ void wait_until_all_kernel(const uint64_t* ivars, size_t n, const int* status, int cmp, const uint64_t* values, uint64_t value) {
  for (size_t i = threadIdx.x; i < n; i += blockDim.x)
    if (!status || !status[i]) wait_until<uint64_t>(ivars + i, cmp, values ? values[i] : value);
}
__global__ void signal_op_kernel(uint64_t* sig, uint64_t value, int op, int pe) { signal_op(sig, value, op, pe); }
__global__ void quiet_kernel() { fence_sys(); }

// ------------------------------------------------------------------ dispatch tables
typedef void (*ReduceLauncher)(int grid, int threads, cudaStream_t s, int team, void* dst, const void* src, size_t n, int algo);

template <class T, int OP, bool RS>
static void launch_reduce(int grid, int threads, cudaStream_t s, int team, void* dst, const void* src, size_t n, int algo) {
  if (RS) reducescatter_kernel<T, OP><<<grid, threads, 0, s>>>(team, (T*)dst, (const T*)src, n, algo);
  else reduce_kernel<T, OP><<<grid, threads, 0, s>>>(team, (T*)dst, (const T*)src, n, algo);
}

template <bool RS>
static ReduceLauncher pick(int dtype, int op) {
#define INT_ROW(T)                                                                                         \
  switch (op) {                                                                                            \
    case OP_AND: return launch_reduce<T, OP_AND, RS>;                                                      \
    case OP_OR: return launch_reduce<T, OP_OR, RS>;                                                        \
    case OP_XOR: return launch_reduce<T, OP_XOR, RS>;                                                      \
    case OP_MIN: return launch_reduce<T, OP_MIN, RS>;                                                      \
    case OP_MAX: return launch_reduce<T, OP_MAX, RS>;                                                      \
    case OP_SUM: return launch_reduce<T, OP_SUM, RS>;                                                      \
    case OP_PROD: return launch_reduce<T, OP_PROD, RS>;                                                    \
  }                                                                                                        \
  return nullptr;
#define FLT_ROW(T)                                                                                         \
  switch (op) {                                                                                            \
    case OP_MIN: return launch_reduce<T, OP_MIN, RS>;                                                      \
    case OP_MAX: return launch_reduce<T, OP_MAX, RS>;                                                      \
    case OP_SUM: return launch_reduce<T, OP_SUM, RS>;                                                      \
    case OP_PROD: return launch_reduce<T, OP_PROD, RS>;                                                    \
  }                                                                                                        \
  return nullptr;
  switch (dtype) {
    case DT_I8: INT_ROW(int8_t)
    case DT_U8: INT_ROW(uint8_t)
    case DT_I16: INT_ROW(int16_t)
    case DT_U16: INT_ROW(uint16_t)
    case DT_I32: INT_ROW(int32_t)
    case DT_U32: INT_ROW(uint32_t)
    case DT_I64: INT_ROW(long long)
    case DT_U64: INT_ROW(unsigned long long)
    case DT_F16: FLT_ROW(__half)
    case DT_BF16: FLT_ROW(__nv_bfloat16)
    case DT_F32: FLT_ROW(float)
    case DT_F64: FLT_ROW(double)
  }
#undef INT_ROW
#undef FLT_ROW
  return nullptr;
}

// ------------------------------------------------------------------ launch geometry
static int clamp_ctas(long want) {
  const long cap = options().MAX_CTAS > 0 ? options().MAX_CTAS : 32;
  long v = want < cap ? want : cap;
  if (v > BSHMEM_SYNC_SLOTS - 2) v = BSHMEM_SYNC_SLOTS - 2;
  return (int)(v < 1 ? 1 : v);
}
// Every CTA runs its own team sync on its own flag slot, so extra CTAs cost no grid-wide step: the
// count only has to cover the latency of the loads and stores in flight.
static int ctas_for(size_t bytes, size_t threshold) {
  if (bytes < threshold) return 1;
  if (bytes < (size_t)256 << 10) return clamp_ctas(4);
  if (bytes < (size_t)1 << 20) return clamp_ctas(8);
  if (bytes < (size_t)4 << 20) return clamp_ctas(16);
  return clamp_ctas(32);
}

// Host-memory heap (no GPU): the data collectives run on the CPU, at once ("on stream" has no meaning there).
static bool host_mode() { return is_initialized() && !rt().have_gpu; }

static int check_team(int team, const char* what) {
  Runtime& r = rt();
  if (!is_initialized()) {
    ERROR_PRINT("%s called before initialisation", what);
    return ST_INVALID_VALUE;
  }
  Team* t = team_get(team);
  if (!t || t->my_pe < 0) {
    ERROR_PRINT("%s: invalid team %d on PE %d", what, team, r.mype);
    return ST_INVALID_VALUE;
  }
  if (!r.have_gpu) {
    ERROR_PRINT("%s needs the GPU heap back end", what);
    return ST_NOT_SUPPORTED;
  }
  return ST_SUCCESS;
}
static int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    ERROR_PRINT("%s: kernel launch failed: %s", what, cudaGetErrorString(e));
    return ST_COLLECTIVE_LAUNCH_FAILED;
  }
  return ST_SUCCESS;
}

int coll_reduce_on_stream(int team, void* dst, const void* src, size_t n, int dtype, int op, cudaStream_t stream, int algo) {
  if (host_mode()) return n ? emul_reduce(team, dst, src, n, dtype, op) : ST_SUCCESS;
  NvtxRange nvtx(NVTX_COLL, "reduce_on_stream");
  int st = check_team(team, "reduce");
  if (st) return st;
  ReduceLauncher f = pick<false>(dtype, op);
  if (!f) return ST_INVALID_VALUE;
  if (n == 0) return ST_SUCCESS;
  const size_t bytes = n * dtype_size(dtype);
  const int threads = (int)std::min<long>(1024, std::max<long>(32, options().REDUCE_NTHREADS));
  f(ctas_for(bytes, (size_t)64 << 10), threads, stream, team, dst, src, n, algo);
  rt().n_coll++;
  return launch_status("reduce");
}

int coll_reducescatter_on_stream(int team, void* dst, const void* src, size_t nreduce, int dtype, int op, cudaStream_t stream, int algo) {
  if (host_mode()) return nreduce ? emul_reducescatter(team, dst, src, nreduce, dtype, op) : ST_SUCCESS;
  NvtxRange nvtx(NVTX_COLL, "reducescatter_on_stream");
  int st = check_team(team, "reducescatter");
  if (st) return st;
  ReduceLauncher f = pick<true>(dtype, op);
  if (!f) return ST_INVALID_VALUE;
  if (nreduce == 0) return ST_SUCCESS;
  const size_t bytes = nreduce * dtype_size(dtype) * team_get(team)->size;
  const int threads = (int)std::min<long>(1024, std::max<long>(32, options().REDUCESCATTER_NTHREADS));
  f(ctas_for(bytes, (size_t)64 << 10), threads, stream, team, dst, src, nreduce, algo);
  rt().n_coll++;
  return launch_status("reducescatter");
}

// ------------------------------------------------------------------ copy-engine variants
// Large alltoall / fcollect / broadcast as one cudaMemcpyAsync per peer into the peer's mapped window, then the
// barrier kernel: the copy engines move the data and no SM is busy meanwhile.  Stream order puts the copies
// before the barrier, whose system-scope fence and flag exchange then tell every member that the data of all
// members has landed.  Off unless NVSHMEM_CE_COLLECTIVES_MIN_BYTES (or nvshmemx_b200_set_ce_collectives) names a
// size; NVSHMEM_DISABLE_CE_COLLECTIVES wins.  (reference: src/host/stream/coll/*: "copy-engine collectives")
static bool ce_wanted(size_t total_bytes, int algo_auto) {
  const size_t min_bytes = rt().ce_min_bytes.load();
  return algo_auto && min_bytes != 0 && total_bytes >= min_bytes && !options().DISABLE_CE_COLLECTIVES;
}
static int ce_copy(void* dst_local_addr, const void* src, size_t bytes, int world_pe, cudaStream_t stream) {
  void* remote = rt().heap->translate(dst_local_addr, world_pe);
  if (!remote) return ST_INVALID_VALUE;
  return cudaMemcpyAsync(remote, src, bytes, cudaMemcpyDeviceToDevice, stream) == cudaSuccess ? ST_SUCCESS : ST_INTERNAL;
}
static int ce_fcollect(Team* t, void* dst, const void* src, size_t block_bytes, cudaStream_t stream) {
  int st = ST_SUCCESS;
  for (int i = 1; i <= t->size && !st; ++i) {  // the member after me first, my own copy last
    const int m = (t->my_pe + i) % t->size;
    st = ce_copy((char*)dst + (size_t)t->my_pe * block_bytes, src, block_bytes, t->members[m], stream);
  }
  return st ? st : coll_barrier_on_stream(t->idx, stream, true);
}
static int ce_alltoall(Team* t, void* dst, const void* src, size_t block_bytes, cudaStream_t stream) {
  int st = ST_SUCCESS;
  for (int i = 1; i <= t->size && !st; ++i) {
    const int m = (t->my_pe + i) % t->size;
    st = ce_copy((char*)dst + (size_t)t->my_pe * block_bytes, (const char*)src + (size_t)m * block_bytes, block_bytes, t->members[m], stream);
  }
  return st ? st : coll_barrier_on_stream(t->idx, stream, true);
}
static int ce_broadcast(Team* t, void* dst, const void* src, size_t bytes, int root, cudaStream_t stream) {
  int st = ST_SUCCESS;
  if (t->my_pe == root)
    for (int i = 1; i <= t->size && !st; ++i) {
      const int m = (t->my_pe + i) % t->size;
      if (m == root && dst == src) continue;
      st = ce_copy(dst, src, bytes, t->members[m], stream);
    }
  return st ? st : coll_barrier_on_stream(t->idx, stream, true);
}

int coll_fcollect_on_stream(int team, void* dst, const void* src, size_t block_bytes, cudaStream_t stream, int algo) {
  if (host_mode()) return block_bytes ? emul_fcollect(team, dst, src, block_bytes) : ST_SUCCESS;
  NvtxRange nvtx(NVTX_COLL, "fcollect_on_stream");
  int st = check_team(team, "fcollect");
  if (st) return st;
  if (block_bytes == 0) return ST_SUCCESS;
  const size_t total = block_bytes * team_get(team)->size;
  if (ce_wanted(total, algo == FC_AUTO) && rt().heap->contains(dst)) {
    rt().n_coll++;
    return ce_fcollect(team_get(team), dst, src, block_bytes, stream);
  }
  const int threads = (int)std::min<long>(1024, std::max<long>(32, options().FCOLLECT_NTHREADS));
  fcollect_kernel<<<ctas_for(total, (size_t)64 << 10), threads, 0, stream>>>(team, dst, src, block_bytes, algo);
  rt().n_coll++;
  return launch_status("fcollect");
}

int coll_alltoall_on_stream(int team, void* dst, const void* src, size_t block_bytes, cudaStream_t stream) {
  if (host_mode()) return block_bytes ? emul_alltoall(team, dst, src, block_bytes) : ST_SUCCESS;
  NvtxRange nvtx(NVTX_COLL, "alltoall_on_stream");
  int st = check_team(team, "alltoall");
  if (st) return st;
  if (block_bytes == 0) return ST_SUCCESS;
  const size_t total = block_bytes * team_get(team)->size;
  if (ce_wanted(total, 1) && rt().heap->contains(dst)) {
    rt().n_coll++;
    return ce_alltoall(team_get(team), dst, src, block_bytes, stream);
  }
  alltoall_kernel<<<ctas_for(total, (size_t)64 << 10), 512, 0, stream>>>(team, dst, src, block_bytes);
  rt().n_coll++;
  return launch_status("alltoall");
}

int coll_broadcast_on_stream(int team, void* dst, const void* src, size_t bytes, int root, cudaStream_t stream, int algo) {
  if (host_mode()) return bytes ? emul_broadcast(team, dst, src, bytes, root) : ST_SUCCESS;
  NvtxRange nvtx(NVTX_COLL, "broadcast_on_stream");
  int st = check_team(team, "broadcast");
  if (st) return st;
  if (root < 0 || root >= team_get(team)->size) return ST_INVALID_VALUE;
  if (bytes == 0) return ST_SUCCESS;
  if (ce_wanted(bytes, algo == BC_AUTO) && rt().heap->contains(dst)) {
    rt().n_coll++;
    return ce_broadcast(team_get(team), dst, src, bytes, root, stream);
  }
  broadcast_kernel<<<ctas_for(bytes, (size_t)64 << 10), 512, 0, stream>>>(team, dst, src, bytes, root, algo);
  rt().n_coll++;
  return launch_status("broadcast");
}

int coll_maxloc_on_stream(int team, void* dst, const void* src, cudaStream_t stream) {
  int st = check_team(team, "maxloc");
  if (st) return st;
  maxloc_kernel<<<1, 32, 0, stream>>>(team, (double2*)dst, (const double2*)src);
  return launch_status("maxloc");
}

int coll_barrier_on_stream(int team, cudaStream_t stream, bool with_quiet) {
  NvtxRange nvtx(NVTX_COLL, with_quiet ? "barrier_on_stream" : "sync_on_stream");
  int st = check_team(team, "barrier");
  if (st) return st;
  const int size = team_get(team)->size;
  const int threads = std::min(1024, (size + 31) / 32 * 32);
  barrier_kernel<<<1, threads, 0, stream>>>(team, kHostSlot, with_quiet ? 1 : 0);
  rt().n_barrier++;
  return launch_status("barrier");
}

// ------------------------------------------------------------------ host-side barrier entry points
static int device_errors_to_status() {
  Runtime& r = rt();
  if (r.status_host && (status_load(&r.status_host->error_bits) & BSHMEM_ERR_WAIT_TIMEOUT)) return ST_INTERNAL;
  return ST_SUCCESS;
}

int host_barrier_team(int team, cudaStream_t stream, bool blocking) {
  Runtime& r = rt();
  if (!r.have_gpu) return emul_team_sync(team);
  // Quiet: earlier non-blocking host puts ran on the internal per-peer streams.
  for (size_t i = 0; i < r.peer_streams.size(); ++i)
    if (r.peer_stream_used[i]) {
      if (blocking) {
        cudaStreamSynchronize(r.peer_streams[i]);
        r.peer_stream_used[i] = false;
      } else {
        cudaEventRecord(r.ev_a, r.peer_streams[i]);
        cudaStreamWaitEvent(stream, r.ev_a, 0);
      }
    }
  int st = coll_barrier_on_stream(team, stream, true);
  if (st) return st;
  if (blocking) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
      ERROR_PRINT("barrier: %s", cudaGetErrorString(e));
      return ST_INTERNAL;
    }
    return device_errors_to_status();
  }
  return ST_SUCCESS;
}

int host_sync_team(int team, cudaStream_t stream, bool blocking) {
  Runtime& r = rt();
  if (!r.have_gpu) return emul_team_sync(team);
  int st = coll_barrier_on_stream(team, stream, false);
  if (st) return st;
  if (blocking) {
    if (cudaStreamSynchronize(stream) != cudaSuccess) return ST_INTERNAL;
    return device_errors_to_status();
  }
  return ST_SUCCESS;
}

int host_barrier_all_blocking() {
  Runtime& r = rt();
  if (r.have_gpu) cudaDeviceSynchronize();
  return host_barrier_team(0, r.stream, true);
}

// ------------------------------------------------------------------ on-stream point-to-point helpers
int p2p_wait_until_on_stream(const void* ivar, int cmp, uint64_t value, int width, bool is_signed, cudaStream_t stream) {
  if (is_signed) wait_until_signed_kernel<<<1, 1, 0, stream>>>((const int64_t*)ivar, cmp, (int64_t)value, width);
  else wait_until_kernel<<<1, 1, 0, stream>>>((const uint64_t*)ivar, cmp, value, width);
  return launch_status("wait_until_on_stream");
}
int p2p_wait_until_all_on_stream(const uint64_t* ivars, size_t n, const int* status, int cmp, const uint64_t* values, uint64_t value, cudaStream_t stream) {
  wait_until_all_kernel<<<1, 128, 0, stream>>>(ivars, n, status, cmp, values, value);
  return launch_status("wait_until_all_on_stream");
}
int p2p_signal_op_on_stream(uint64_t* sig, uint64_t value, int op, int pe, cudaStream_t stream) {
  signal_op_kernel<<<1, 1, 0, stream>>>(sig, value, op, pe);
  return launch_status("signal_op_on_stream");
}
int p2p_quiet_on_stream(cudaStream_t stream) {
  quiet_kernel<<<1, 1, 0, stream>>>();
  return launch_status("quiet_on_stream");
}

}  // namespace bshmem
