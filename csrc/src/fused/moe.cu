// Expert-parallel MoE dispatch and combine for sm_100a over NVLink peer memory.
//
// dispatch (one cooperative kernel, persistent CTAs of 256 threads):
//   A  histogram of the K expert ids of every token (shared-memory bins, then global atomics)
//   B  CTA 0 stores this PE's E counts into row `rank` of every PE's count matrix and runs a
//      cross-PE barrier; a grid barrier releases the other CTAs
//   C  every CTA derives, from the complete [npes, E] matrix, the first row of each expert's
//      segment that belongs to this PE as a source: rows of a receive buffer are ordered by
//      local expert, then by source PE, so the expert GEMMs read contiguous groups
//   D  one CTA per token: the row is staged in shared memory once (and quantised once to fp8 with
//      1x128 fp32 scales when asked), each of its K slots takes the next row of its segment with an
//      atomic cursor, and the row is pushed with 16-byte stores to the owning PE.  With `dup_src` a row
//      crosses NVLink once per destination PE: the first of the token's slots on a PE carries the payload,
//      the others only the number of that row
//   E  grid barrier, then a cross-PE barrier: every PE's rows have landed
//   F  (with `dup_src`) every PE copies the rows that arrived by number from their first row, locally
// combine (one cooperative kernel): cross-PE barrier on entry (expert outputs are final), then one CTA
// per token pulls its K rows with 16-byte loads from the owners, multiplies by the routing weights in
// fp32, rounds once to bf16; a cross-PE barrier on exit lets the owners reuse their buffers.
// All waits are bounded and report through `error_flag`; nothing traps.
// (reference for the capability: examples/moe_shuffle.cu, an fp32 dispatch-only all-to-all-v)
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/bshmem/moe.h"

namespace bshmem {
namespace moe {

constexpr int THREADS = 256;

struct Scratch {                 // local device memory, zeroed by the host before each dispatch
  unsigned int grid_bar;         // arrivals at grid barriers (monotonic within a launch)
  unsigned int pad[63];
  int send_count[BSHMEM_MOE_MAX_EXPERTS];   // pairs this PE sends to each expert
  int cursor[BSHMEM_MOE_MAX_EXPERTS];       // next free position inside my segment of each expert
};

struct DispatchParams {
  bshmem_moe_dispatch_args_t a;
  uint64_t wait_limit_ns;
};
struct CombineParams {
  bshmem_moe_combine_args_t a;
  uint64_t wait_limit_ns;
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid barrier over co-resident CTAs (cooperative launch).  `phase` counts barriers of this launch; the
// counter starts at zero.  Returns false after the wait bound.
__device__ bool grid_barrier(unsigned* counter, unsigned& phase, uint64_t limit_ns, int* error_flag) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    ++phase;
    __threadfence();
    atomicAdd(counter, 1u);
    const unsigned target = phase * gridDim.x;
    const uint64_t start = timer_ns();
    int ok = 1;
    unsigned spins = 0;
    while (ld_acquire_gpu_u32(counter) < target) {
      if ((++spins & 63) == 0 && timer_ns() - start > limit_ns) {
        atomicOr(error_flag, BSHMEM_MOE_ERRBIT_TIMEOUT);
        ok = 0;
        break;
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}

// Cross-PE barrier run by the first `npes` threads of one CTA: store `value` into slot `rank` of row
// `row` of every PE's flag block, wait until every slot of my row holds at least `value`.
__device__ bool pe_barrier(uint64_t* const* flags, int row, int rank, int npes, uint64_t value, uint64_t limit_ns, int* error_flag) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < npes) {
    const int q = threadIdx.x;
    __threadfence_system();
    if (q != rank) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flags[q] + row * npes + rank), "l"(value) : "memory");
    if (q != rank) {
      const uint64_t* mine = flags[rank] + row * npes + q;
      const uint64_t start = timer_ns();
      unsigned spins = 0;
      while (ld_acquire_sys_u64(mine) < value) {
        if ((++spins & 31) == 0) {
          if (timer_ns() - start > limit_ns) {
            atomicOr(error_flag, BSHMEM_MOE_ERRBIT_TIMEOUT);
            ok_s = 0;
            break;
          }
          __nanosleep(64);
        }
      }
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__global__ void __launch_bounds__(THREADS) dispatch_kernel(const __grid_constant__ DispatchParams P) {
  const bshmem_moe_dispatch_args_t& a = P.a;
  extern __shared__ __align__(16) uint8_t smem[];
  const int T = a.T, H = a.H, K = a.K, E = a.E, npes = a.npes, rank = a.rank;
  const int EL = E / npes;
  Scratch* sc = (Scratch*)a.scratch;
  unsigned phase = 0;
  int* s_bins = (int*)smem;                     // [E] histogram bins, later my segment starts; [E] more for totals
  __shared__ int s_row[THREADS], s_dest[THREADS];  // slots of one chunk of tokens: [token in chunk][choice]
  __shared__ int s_first[THREADS];                 // -1: this slot carries the payload; else the row (same PE) that does
  const bool dedup = a.dup_src[rank] != nullptr;

  // ---- A: histogram
  for (int e = threadIdx.x; e < E; e += THREADS) s_bins[e] = 0;
  __syncthreads();
  for (long i = (long)blockIdx.x * THREADS + threadIdx.x; i < (long)T * K; i += (long)gridDim.x * THREADS) {
    const int e = a.topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&s_bins[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += THREADS)
    if (s_bins[e]) atomicAdd(&sc->send_count[e], s_bins[e]);
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;

  // ---- B: publish my counts to every PE, cross-PE barrier
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < E * npes; i += THREADS) {
      const int q = i / E, e = i % E;
      a.counts[q][rank * E + e] = sc->send_count[e];
    }
    __syncthreads();
    pe_barrier(a.flags, 0, rank, npes, a.epoch, P.wait_limit_ns, a.error_flag);
  }
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;

  // ---- C: where my rows start on each owner.  Rows of PE d's buffer: for le in [0, EL): for s in [0, npes): count[s][d*EL+le] rows.
  // Per expert: rows from all PEs (s_tot) and rows from the PEs before me (s_bins); then a prefix over
  // the experts of one owner, from shared memory.
  const int* cm = a.counts[rank];
  int* s_tot = s_bins + E;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += THREADS) {
    int tot = 0, pre = 0;
    for (int s = 0; s < npes; ++s) {
      const int c = __ldcg(&cm[s * E + e]);
      tot += c;
      if (s < rank) pre += c;
    }
    s_tot[e] = tot;
    s_bins[e] = pre;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += THREADS) {
    const int first = (e / EL) * EL;
    int start = s_bins[e];
    for (int l2 = first; l2 < e; ++l2) start += s_tot[l2];
    s_bins[e] = start;  // only this thread reads or writes s_bins[e] in this loop
  }
  if (blockIdx.x == 0) {  // receiver-side description of my own buffer
    for (int le = threadIdx.x; le <= EL; le += THREADS) {
      int start = 0;
      for (int l2 = 0; l2 < le; ++l2) start += s_tot[rank * EL + l2];
      a.expert_offsets[le] = start;
      if (le < EL && a.src_offsets) {
        int run = start;
        for (int s = 0; s < npes; ++s) {
          a.src_offsets[le * npes + s] = run;
          run += __ldcg(&cm[s * E + rank * EL + le]);
        }
      }
    }
  }

  // ---- D: push rows.  The slots of a whole chunk of this CTA's tokens are claimed first (one atomic per
  // (token, choice) pair, all in flight together); after that each token moves from global memory through
  // registers to its K destinations with no CTA-wide synchronisation, so that the loads of one token
  // overlap the stores of the one before.
  const int row_bytes = a.payload == BSHMEM_MOE_FP8_E4M3 ? H : H * 2;
  const int nscale = H / BSHMEM_MOE_QUANT_BLOCK;
  const int per_chunk = THREADS / K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int base = 0; (long)blockIdx.x + (long)base * gridDim.x < T; base += per_chunk) {
    __syncthreads();  // the previous chunk's slots are no longer read (and s_bins is final on the first pass)
    {
      const int i = threadIdx.x / K, k = threadIdx.x % K;
      const long t = (long)blockIdx.x + (long)(base + i) * gridDim.x;
      if (i < per_chunk && t < T) {
        const int e = a.topk_idx[(size_t)t * K + k];
        int row = -1, dest = 0;
        if (e >= 0 && e < E) {
          const int pos = atomicAdd(&sc->cursor[e], 1);
          row = s_bins[e] + pos;
          dest = e / EL;
          if (row >= a.cap_rows) {
            atomicOr(a.error_flag, BSHMEM_MOE_ERRBIT_OVERFLOW);
            row = -1;
          }
        }
        s_row[i * K + k] = row;
        s_dest[i * K + k] = dest;
        a.slot_map[(size_t)t * K + k] = row;
      }
    }
    __syncthreads();
    {
      // Which slot of the token carries the payload to each destination PE: the first valid one.
      const int i = threadIdx.x / K, k = threadIdx.x % K;
      const long t = (long)blockIdx.x + (long)(base + i) * gridDim.x;
      if (i < per_chunk && t < T) {
        int first = -1;
        const int row = s_row[i * K + k], dest = s_dest[i * K + k];
        if (dedup && row >= 0) {
          for (int j = 0; j < k; ++j)
            if (s_row[i * K + j] >= 0 && s_dest[i * K + j] == dest) { first = s_row[i * K + j]; break; }
          a.dup_src[dest][row] = first;  // every row is written by its sender: -1 = payload follows, else copy from `first`
        }
        s_first[i * K + k] = first;
      }
    }
    __syncthreads();
    for (int i = 0; i < per_chunk; ++i) {
      const long t = (long)blockIdx.x + (long)(base + i) * gridDim.x;
      if (t >= T) break;
      const int* rows = s_row + i * K;
      const int* dests = s_dest + i * K;
      const int* firsts = s_first + i * K;
      if (a.payload == BSHMEM_MOE_FP8_E4M3) {
        // Eight lanes per 128-value block, 16 values per lane: a warp quantises four blocks at a time and
        // stores 16 bytes per lane (512 contiguous bytes per warp and destination).  absmax over the eight
        // lanes by shuffles, scale = amax / 448.  Two rounds of loads are in flight before the first store.
        const uint4* xrow = (const uint4*)a.x + (size_t)t * (H / 8);
        constexpr int WARPS = THREADS / 32;
        const int sub = lane >> 3, part = lane & 7;  // block within the warp's four, 16-value piece within the block
        const int ngroups = (nscale + 3) / 4;
        for (int q0 = warp; q0 < ngroups; q0 += 2 * WARPS) {
          uint4 raw[2][2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int g = (q0 + u * WARPS) * 4 + sub;
            if (q0 + u * WARPS < ngroups && g < nscale) {
              raw[u][0] = xrow[g * 16 + part * 2];
              raw[u][1] = xrow[g * 16 + part * 2 + 1];
            } else {
              raw[u][0] = raw[u][1] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (q0 + u * WARPS >= ngroups) break;  // uniform over the warp
            const int g = (q0 + u * WARPS) * 4 + sub;
            float f[16];
            const __nv_bfloat162* h = (const __nv_bfloat162*)raw[u];
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float2 v = __bfloat1622float2(h[e]);
              f[2 * e] = v.x;
              f[2 * e + 1] = v.y;
              amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float scale = fmaxf(amax, 1e-10f) / 448.0f;
            const float inv = 1.0f / scale;
            uint4 q16;
            uint32_t* qw = (uint32_t*)&q16;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * e] * inv, f[4 * e + 1] * inv), __NV_SATFINITE, __NV_E4M3);
              const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * e + 2] * inv, f[4 * e + 3] * inv), __NV_SATFINITE, __NV_E4M3);
              qw[e] = (uint32_t)lo | ((uint32_t)hi << 16);
            }
            if (g < nscale) {
              for (int j = 0; j < K; ++j) {
                const int row = rows[j];
                if (row < 0 || firsts[j] >= 0) continue;
                ((uint4*)((uint8_t*)a.recv_x[dests[j]] + (size_t)row * row_bytes))[g * 8 + part] = q16;
                if (part == 0) a.recv_scale[dests[j]][(size_t)row * nscale + g] = scale;
              }
            }
          }
        }
      } else {
        const uint4* xrow = (const uint4*)a.x + (size_t)t * (H / 8);
        const int nvec = H / 8;
        for (int c0 = threadIdx.x; c0 < nvec; c0 += 4 * THREADS) {
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + u * THREADS < nvec) v[u] = xrow[c0 + u * THREADS];
          for (int j = 0; j < K; ++j) {
            const int row = rows[j];
            if (row < 0 || firsts[j] >= 0) continue;
            uint4* dst = (uint4*)((uint8_t*)a.recv_x[dests[j]] + (size_t)row * row_bytes);
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (c0 + u * THREADS < nvec) dst[c0 + u * THREADS] = v[u];
          }
        }
      }
    }
  }

  // ---- E: all my rows are out; meet every PE
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;
  if (blockIdx.x == 0) pe_barrier(a.flags, 1, rank, npes, a.epoch, P.wait_limit_ns, a.error_flag);
  if (!dedup) return;

  // ---- F: rows that arrived as a row number are copied from that row (always a payload row), locally
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;
  int total = 0;
  for (int le = 0; le < EL; ++le) total += s_tot[rank * EL + le];
  if (total > a.cap_rows) total = a.cap_rows;
  const int* dup = a.dup_src[rank];
  uint8_t* mine = (uint8_t*)a.recv_x[rank];
  const int nvec = row_bytes / 16;
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    const int from = __ldcg(dup + r);
    if (from < 0 || from >= total) continue;
    const uint4* src = (const uint4*)(mine + (size_t)from * row_bytes);
    uint4* dst = (uint4*)(mine + (size_t)r * row_bytes);
    for (int c = threadIdx.x; c < nvec; c += THREADS) dst[c] = __ldcg(src + c);
    if (a.payload == BSHMEM_MOE_FP8_E4M3)
      for (int g = threadIdx.x; g < nscale; g += THREADS) a.recv_scale[rank][(size_t)r * nscale + g] = __ldcg(&a.recv_scale[rank][(size_t)from * nscale + g]);
  }
}

// Weighted sum of up to KT expert rows into one output row.  Row pointers and weights sit in registers;
// for every 16-byte column block the KT loads are issued before the first is consumed.
template <int KT>
__device__ __forceinline__ void combine_token(const uint8_t* const* src, const float* wt, int K, uint4* out_row, int nvec) {
  const uint4* p[KT];
  float w[KT];
#pragma unroll
  for (int j = 0; j < KT; ++j) {
    const bool on = j < K && src[j] != nullptr;
    p[j] = on ? (const uint4*)src[j] : nullptr;
    w[j] = on ? wt[j] : 0.f;
  }
  for (int c = threadIdx.x; c < nvec; c += THREADS) {
    uint4 v[KT];
#pragma unroll
    for (int j = 0; j < KT; ++j) v[j] = p[j] ? p[j][c] : make_uint4(0u, 0u, 0u, 0u);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < KT; ++j) {
      const __nv_bfloat162* h = (const __nv_bfloat162*)&v[j];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += w[j] * f.x;
        acc[2 * q + 1] += w[j] * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = (__nv_bfloat162*)&o;
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    out_row[c] = o;
  }
}

template <int KT>
__global__ void __launch_bounds__(THREADS, KT <= 8 ? 3 : 2) combine_kernel(const __grid_constant__ CombineParams P) {
  const bshmem_moe_combine_args_t& a = P.a;
  const int T = a.T, H = a.H, K = a.K, E = a.E, npes = a.npes, rank = a.rank;
  const int EL = E / npes;
  Scratch* sc = (Scratch*)a.scratch;
  unsigned phase = 0;
  __shared__ const uint8_t* s_src[THREADS];  // one chunk of this CTA's tokens: [token in chunk][choice]
  __shared__ float s_w[THREADS];
  if (blockIdx.x == 0) pe_barrier(a.flags, 2, rank, npes, a.epoch, P.wait_limit_ns, a.error_flag);
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;
  const int per_chunk = THREADS / K;
  for (int base = 0; (long)blockIdx.x + (long)base * gridDim.x < T; base += per_chunk) {
    __syncthreads();
    {
      // Sources and weights of a whole chunk of tokens are looked up at once, so that the token loop
      // below runs without CTA-wide synchronisation.
      const int i = threadIdx.x / K, k = threadIdx.x % K;
      const long t = (long)blockIdx.x + (long)(base + i) * gridDim.x;
      if (i < per_chunk && t < T) {
        const int e = a.topk_idx[(size_t)t * K + k];
        const int row = a.slot_map[(size_t)t * K + k];
        const bool ok = e >= 0 && e < E && row >= 0;
        s_src[i * K + k] = ok ? (const uint8_t*)a.y[e / EL] + (size_t)row * H * 2 : nullptr;
        s_w[i * K + k] = ok ? a.topk_weight[(size_t)t * K + k] : 0.f;
      }
    }
    __syncthreads();
    for (int i = 0; i < per_chunk; ++i) {
      const long t = (long)blockIdx.x + (long)(base + i) * gridDim.x;
      if (t >= T) break;
      uint4* out_row = (uint4*)a.out + (size_t)t * (H / 8);
      combine_token<KT>(s_src + i * K, s_w + i * K, K, out_row, H / 8);
    }
  }
  if (!grid_barrier(&sc->grid_bar, phase, P.wait_limit_ns, a.error_flag)) return;
  if (blockIdx.x == 0) pe_barrier(a.flags, 3, rank, npes, a.epoch, P.wait_limit_ns, a.error_flag);
}

static size_t dispatch_smem(int E, int) { return (size_t)E * 8 + 16; }  // two int arrays of E entries; rows go through registers

// Cooperative grid: as many CTAs as are co-resident, at most one per token.
template <class Kernel>
static int coop_grid(Kernel k, size_t smem, int want, int max_ctas, int* grid_out) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return BSHMEM_MOE_ERR_DRIVER;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, THREADS, smem) != cudaSuccess || per_sm < 1) return BSHMEM_MOE_ERR_DRIVER;
  int grid = per_sm * sms;
  if (grid > want) grid = want;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid < 1) grid = 1;
  *grid_out = grid;
  return 0;
}

}  // namespace moe
}  // namespace bshmem

using namespace bshmem::moe;

extern "C" size_t bshmem_moe_scratch_bytes(int) { return sizeof(Scratch); }

static int check_common(int T, int H, int K, int E, int rank, int npes) {
  if (npes < 1 || npes > BSHMEM_MOE_MAX_PES || rank < 0 || rank >= npes) return BSHMEM_MOE_ERR_ARGS;
  if (T <= 0 || K < 1 || K > BSHMEM_MOE_MAX_TOPK || E < npes || E > BSHMEM_MOE_MAX_EXPERTS || E % npes) return BSHMEM_MOE_ERR_SHAPE;
  if (H <= 0 || H % BSHMEM_MOE_QUANT_BLOCK) return BSHMEM_MOE_ERR_SHAPE;  // rows are moved in 16-byte pieces and quantised in blocks of 128
  return 0;
}

extern "C" int bshmem_moe_dispatch(const bshmem_moe_dispatch_args_t* a, cudaStream_t stream) {
  if (!a || !a->x || !a->topk_idx || !a->slot_map || !a->expert_offsets || !a->scratch || !a->error_flag) return BSHMEM_MOE_ERR_ARGS;
  int st = check_common(a->T, a->H, a->K, a->E, a->rank, a->npes);
  if (st) return st;
  for (int q = 0; q < a->npes; ++q)
    if (!a->recv_x[q] || !a->counts[q] || !a->flags[q] || (a->payload == BSHMEM_MOE_FP8_E4M3 && !a->recv_scale[q])) return BSHMEM_MOE_ERR_ARGS;
  DispatchParams P;
  P.a = *a;
  P.wait_limit_ns = a->wait_limit_ms ? (uint64_t)a->wait_limit_ms * 1000000ull : 10000000000ull;
  const size_t smem = dispatch_smem(a->E, a->H);
  int grid = 0;
  st = coop_grid(dispatch_kernel, smem, a->T, a->max_ctas, &grid);
  if (st) return st;
  if (cudaMemsetAsync(a->scratch, 0, sizeof(Scratch), stream) != cudaSuccess) return BSHMEM_MOE_ERR_DRIVER;
  void* params[] = {(void*)&P};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)dispatch_kernel, dim3(grid), dim3(THREADS), params, smem, stream);
  if (e != cudaSuccess) {
    fprintf(stderr, "bshmem_moe_dispatch: launch failed: %s\n", cudaGetErrorString(e));
    return BSHMEM_MOE_ERR_DRIVER;
  }
  return 0;
}

extern "C" int bshmem_moe_combine(const bshmem_moe_combine_args_t* a, cudaStream_t stream) {
  if (!a || !a->topk_idx || !a->topk_weight || !a->slot_map || !a->out || !a->scratch || !a->error_flag) return BSHMEM_MOE_ERR_ARGS;
  int st = check_common(a->T, a->H, a->K, a->E, a->rank, a->npes);
  if (st) return st;
  for (int q = 0; q < a->npes; ++q)
    if (!a->y[q] || !a->flags[q]) return BSHMEM_MOE_ERR_ARGS;
  CombineParams P;
  P.a = *a;
  P.wait_limit_ns = a->wait_limit_ms ? (uint64_t)a->wait_limit_ms * 1000000ull : 10000000000ull;
  int grid = 0;
  // Two builds of the kernel: up to 8 choices per token (fewer registers, three CTAs per SM) and up to 16.
  const void* kernel = a->K <= 8 ? (const void*)combine_kernel<8> : (const void*)combine_kernel<BSHMEM_MOE_MAX_TOPK>;
  st = a->K <= 8 ? coop_grid(combine_kernel<8>, 0, a->T, a->max_ctas, &grid) : coop_grid(combine_kernel<BSHMEM_MOE_MAX_TOPK>, 0, a->T, a->max_ctas, &grid);
  if (st) return st;
  if (cudaMemsetAsync(a->scratch, 0, 256, stream) != cudaSuccess) return BSHMEM_MOE_ERR_DRIVER;  // the grid-barrier counter
  void* params[] = {(void*)&P};
  cudaError_t e = cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(THREADS), params, 0, stream);
  if (e != cudaSuccess) {
    fprintf(stderr, "bshmem_moe_combine: launch failed: %s\n", cudaGetErrorString(e));
    return BSHMEM_MOE_ERR_DRIVER;
  }
  return 0;
}

// ------------------------------------------------------------------ dispatch without any allocation
// Single-PE dispatch whose scratch is a fixed array inside this library (see bshmem/moe_noalloc.h
// for who needs that and the rules of use).  In host code the array's name is only a handle; the
// address a kernel can use comes from cudaGetSymbolAddress, looked up once per GPU.
#include <limits.h>

#include <atomic>

#include "../../include/bshmem/moe_noalloc.h"

namespace {

struct NoAllocBlock {
  bshmem::moe::Scratch scratch;                    // counters + grid-barrier word (cleared every call)
  int counts[BSHMEM_MOE_NOALLOC_MAX_EXPERTS];      // the 1 x E count matrix
  uint64_t flags[4];                               // cross-PE barrier rows (unused with one PE, must exist)
  int error_flag;                                  // used when the caller passes none
  int pad[7];
};
static_assert(sizeof(NoAllocBlock) <= BSHMEM_MOE_NOALLOC_SCRATCH_BYTES, "documented scratch size is too small");

static __device__ __align__(256) unsigned char g_noalloc_block[BSHMEM_MOE_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::atomic<NoAllocBlock*> g_noalloc_addr[kMaxDevices];  // device address of the array, per GPU ordinal (any host thread may fill it)

// Device address of the array on the current GPU, looked up on first use.
static int noalloc_block(NoAllocBlock** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return BSHMEM_MOE_ERR_DRIVER;
  NoAllocBlock* blk = g_noalloc_addr[dev].load(std::memory_order_acquire);
  if (!blk) {  // first call on this GPU (it is the current device): resolve the array's device address
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_block);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "bshmem_moe_dispatch_local_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return BSHMEM_MOE_ERR_DRIVER;
    }
    blk = (NoAllocBlock*)p;
    g_noalloc_addr[dev].store(blk, std::memory_order_release);  // two threads racing here store the same address
  }
  *out = blk;
  return BSHMEM_MOE_OK;
}

}  // namespace

extern "C" int bshmem_moe_dispatch_local_noalloc(const void* x, const int* topk_idx, int T, int H, int K, int E, void* recv_x, int* slot_map, int* expert_offsets,
                                                 int* error_flag, cudaStream_t stream) {
  if (!x || !topk_idx || !recv_x || !slot_map || !expert_offsets) return BSHMEM_MOE_ERR_ARGS;
  if (E > BSHMEM_MOE_NOALLOC_MAX_EXPERTS || E < 1 || K < 1 || K > BSHMEM_MOE_MAX_TOPK || T < 1 || H < 1 || H % BSHMEM_MOE_QUANT_BLOCK) {
    fprintf(stderr, "bshmem_moe_dispatch_local_noalloc: unsupported size (T=%d H=%d K=%d E=%d): at most %d experts and top-%d, H a multiple of %d\n", T, H, K, E,
            BSHMEM_MOE_NOALLOC_MAX_EXPERTS, BSHMEM_MOE_MAX_TOPK, BSHMEM_MOE_QUANT_BLOCK);
    return BSHMEM_MOE_ERR_SHAPE;
  }
  if ((long long)T * K > INT_MAX) {  // row numbers are 32-bit
    fprintf(stderr, "bshmem_moe_dispatch_local_noalloc: T * K = %lld rows do not fit 32-bit row numbers\n", (long long)T * K);
    return BSHMEM_MOE_ERR_SHAPE;
  }
  NoAllocBlock* blk = nullptr;
  int bst = noalloc_block(&blk);
  if (bst) return bst;
  // The block keeps what the previous call left: clear the counters, the barrier word, the flags and the built-in error word.
  if (cudaMemsetAsync(blk, 0, sizeof(NoAllocBlock), stream) != cudaSuccess) return BSHMEM_MOE_ERR_DRIVER;

  DispatchParams P;
  memset(&P, 0, sizeof(P));
  bshmem_moe_dispatch_args_t& a = P.a;
  a.T = T; a.H = H; a.K = K; a.E = E; a.rank = 0; a.npes = 1;
  a.payload = BSHMEM_MOE_BF16;
  a.cap_rows = T * K;
  a.epoch = 1;
  a.error_flag = error_flag ? error_flag : &blk->error_flag;
  a.x = x;
  a.topk_idx = topk_idx;
  a.recv_x[0] = recv_x;
  a.slot_map = slot_map;
  a.expert_offsets = expert_offsets;
  a.src_offsets = nullptr;
  a.counts[0] = blk->counts;
  a.flags[0] = blk->flags;
  a.scratch = &blk->scratch;
  P.wait_limit_ns = 10000000000ull;
  const size_t smem = dispatch_smem(E, H);
  int grid = 0;
  int st = coop_grid(dispatch_kernel, smem, T, 0, &grid);
  if (st) return st;
  void* params[] = {(void*)&P};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)dispatch_kernel, dim3(grid), dim3(THREADS), params, smem, stream);
  if (e != cudaSuccess) {
    fprintf(stderr, "bshmem_moe_dispatch_local_noalloc: launch failed: %s\n", cudaGetErrorString(e));
    return BSHMEM_MOE_ERR_DRIVER;
  }
  return BSHMEM_MOE_OK;
}

extern "C" int bshmem_moe_noalloc_error_bits(cudaStream_t stream, int* bits) {
  if (!bits) return BSHMEM_MOE_ERR_ARGS;
  NoAllocBlock* blk = nullptr;
  int st = noalloc_block(&blk);
  if (st) return st;
  if (cudaMemcpyAsync(bits, &blk->error_flag, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return BSHMEM_MOE_ERR_DRIVER;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_MOE_OK : BSHMEM_MOE_ERR_DRIVER;
}
