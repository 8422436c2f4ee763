// Pieces shared by the two variants of the fused GEMM kernel (one CTA per tile, and CTA pairs that
// share a 256x256 tile): parameter block, tile order, bounded flag wait, the all-gather sender and
// the host helper that encodes TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/bshmem/fused.h"
#include "../../include/bshmem/tcgen05.cuh"
#include "../../include/bshmem/nvls.cuh"

namespace bshmem {
using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int A_STAGE = BM * BK * 2;
constexpr int EPI_COLS = 64, EPI_BUF = BM * EPI_COLS * 2, EPI_BUFS = 2;
constexpr int TMEM_COLS = 512, ACC_COLS = BN;
constexpr int NTHREADS = 256, EPI_THREADS = 128, EPI_WARP0 = 4;
constexpr int AUX_WARP0 = 2, AUX_THREADS = 64;   // warps 2 and 3: switch-side reduction (RS / AR) or shard sender (AG)
constexpr int SMEM_TILES = 4 * (A_STAGE + BN * BK * 2) + EPI_BUFS * EPI_BUF;  // 4 stages of a 128 x 256 tile = 6 stages of a pair's halves
constexpr int MAX_GROUPS = 256;                   // grouped mode: experts (row groups) per call
constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 256 /*barriers*/ + (MAX_GROUPS + 4) * 4 /*grouped mode: tile prefix sums*/;

struct alignas(64) FusedParams {
  CUtensorMap tmA, tmB;
  CUtensorMap tmOut[BSHMEM_FUSED_MAX_PES];   // PLAIN/RS/AG: [0] is the local output; AR: output of each PE
  CUtensorMap tmRecv[BSHMEM_FUSED_MAX_PES];  // RS/AR, push path: my slot in the receive buffer of each PE
  CUtensorMap tmStage;                       // RS/AR, switch path: this PE's staging buffer [M][N] of partial tiles
  const char* stage_mc;                      // multicast alias of the staging buffer (non-null selects the switch path)
  char* out_local;                           // RS switch path: this PE's [M/npes][N] output
  const __nv_bfloat16* recv_local;           // [npes][M/npes][N] partials received from each PE
  uint64_t* flags_local;                     // [npes][tiles per PE]
  uint64_t* flags_peer[BSHMEM_FUSED_MAX_PES];
  const char* ag_src;                        // my shard inside my gathered buffer
  char* ag_dst[BSHMEM_FUSED_MAX_PES];        // the same shard inside each PE's gathered buffer
  uint64_t* ag_flags_local;                  // [npes][m-tiles per shard]: rows of the 128-row block that have landed (x epoch)
  uint64_t* ag_flags_peer[BSHMEM_FUSED_MAX_PES];
  char* out_mc;                              // AR: multicast alias of the output (null: per-PE stores)
  int* error_flag;
  uint64_t epoch, wait_limit_ns;
  int M, N, K, rank, npes, mode;
  int ag_external;                           // AG: the shards are pushed by the caller (copy engines); flag [peer][0] = epoch when a shard is complete
  int act;                                   // BSHMEM_FUSED_ACT_*: applied to the fp32 result in the epilogue (PLAIN / AG)
  const int* group_offsets;                  // GROUPED: device array [groups + 1], rows of group g are [offsets[g], offsets[g + 1])
  int groups, group_n;                       // GROUPED: number of groups; rows of B (output columns) per group
  int red_rows;                              // switch path: rows per work item of the reducing warps (16 or 32)
  int sw_reduce;                             // RS/AR: partial tiles stay local and the owner fetches their sum through the switch
};

struct TileInfo {
  int a_row, b_row;     // row coordinates of the tile's operands: first row of A, first row of B (the CTA pair adds its half)
  int valid_rows;       // rows of the tile that exist (BM except in the last tile of a group, GROUPED mode)
  int m_tile, n_tile;   // position in the full output
  int peer;             // RS/AR: PE that owns the rows; AG: PE whose shard holds the rows
  int m_local;          // m-tile index inside that PE's block of rows
  int idx_in_peer;      // tile number inside the block (flag index)
};

// Tile order.  Blocks of rows are visited peer by peer (RS/AR: rank+1, rank+2, …, own last; AG: own, rank-1, …);
// inside a block m runs fastest so that concurrently running CTAs share B tiles through L2.
// Switch path of RS/AR: every PE walks the output in the same order (m fastest over all rows, then n), so that the
// partials of a tile are produced at about the same time everywhere and its owner can reduce it right away; owners
// alternate every M/npes rows, so the reduction traffic is spread evenly over the PEs and over the run.
__host__ __device__ __forceinline__ TileInfo tile_info_base(const FusedParams& p, int t);
__host__ __device__ __forceinline__ TileInfo tile_info(const FusedParams& p, int t) {
  TileInfo ti = tile_info_base(p, t);
  ti.a_row = ti.m_tile * BM;
  ti.b_row = ti.n_tile * BN;
  ti.valid_rows = BM;
  return ti;
}
// GROUPED mode (C rows of group g = A rows of group g times B_g^T, group boundaries in device memory): `prefix[g]` is
// the number of tiles of the groups before g (built once per CTA in shared memory).  Inside a group the 128-row
// blocks run fastest, then the column blocks.  The last block of a group may be short: its operand tile still loads
// 128 rows (whatever follows the group; rows past the end of A read as zero) and only `valid_rows` rows are stored.
__device__ __forceinline__ TileInfo grouped_tile_info(const FusedParams& p, const int* prefix, int t) {
  int lo = 0, hi = p.groups;  // find g with prefix[g] <= t < prefix[g + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= t) lo = mid;
    else hi = mid;
  }
  const int g = lo, local = t - prefix[g];
  const int r0 = p.group_offsets[g], r1 = p.group_offsets[g + 1];
  const int mblocks = (r1 - r0 + BM - 1) / BM;
  TileInfo ti;
  ti.peer = g;
  ti.m_local = local % mblocks;
  ti.n_tile = local / mblocks;
  ti.m_tile = 0;
  ti.idx_in_peer = local;
  ti.a_row = r0 + ti.m_local * BM;
  ti.b_row = g * p.group_n + ti.n_tile * BN;
  ti.valid_rows = r1 - ti.a_row < BM ? r1 - ti.a_row : BM;
  return ti;
}
__host__ __device__ __forceinline__ TileInfo tile_info_base(const FusedParams& p, int t) {
  const int tiles_n = p.N / BN;
  const int tmr = (p.M / p.npes) / BM;
  const int per_peer = tmr * tiles_n;
  TileInfo ti;
  if (p.sw_reduce) {
    const int tiles_m = tmr * p.npes;
    ti.m_tile = t % tiles_m;
    ti.n_tile = t / tiles_m;
    ti.peer = ti.m_tile / tmr;
    ti.m_local = ti.m_tile % tmr;
    ti.idx_in_peer = ti.n_tile * tmr + ti.m_local;
    return ti;
  }
  const int o = t / per_peer, within = t % per_peer;
  if (p.mode == BSHMEM_FUSED_AG) ti.peer = (p.rank - o + p.npes) % p.npes;
  else ti.peer = (p.rank + 1 + o) % p.npes;
  ti.m_local = within % tmr;
  ti.n_tile = within / tmr;
  ti.m_tile = ti.peer * tmr + ti.m_local;
  ti.idx_in_peer = within;
  return ti;
}

// GELU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), with the hardware tanh approximation.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ bool wait_flag_ge(const uint64_t* flag, uint64_t want, uint64_t limit_ns, volatile int* abort_flag) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
  if (v >= want) return true;
  const uint64_t start = timer_ns();
  uint32_t spins = 0;
  for (;;) {
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= want) return true;
    if ((++spins & 31) == 0) {
      if (*abort_flag) return false;
      if (timer_ns() - start > limit_ns) {
        *abort_flag = 1;
        return false;
      }
      __nanosleep(64);
    }
  }
}

// ------------------------------------------------------------------ auxiliary warps (warps 2 and 3 of every CTA)
__device__ __forceinline__ void aux_bar_sync() { named_bar_sync(2, AUX_THREADS); }

// MODE_AG, in-kernel sender: the 64 auxiliary threads of every CTA copy part of this PE's shard into every peer's
// gathered buffer with 16-byte loads and stores, nearest peer first.  The shard is cut into units (a row, or a
// power-of-two fraction of one when there are more CTAs than rows in a block) and the units of every 128-row block
// are dealt round-robin to the CTAs.  After a peer's copy a CTA makes its stores visible (one barrier of the 64
// threads, one system-scope fence by one thread: a fence drains the CTA's stores in flight, so it is paid once per
// peer and not per block) and adds the number of units it delivered to each block's arrival counter on that peer; a
// block is complete when its counter has grown by `units_per_block`.
// Loads issued by these warps share the L2-to-SM fabric with the operand traffic of the tensor cores and see long
// latencies, so this path moves a few hundred GB/s per GPU at best; the default is therefore the external sender
// (FusedParams::ag_external: copy engines push the shards and set one flag per shard, see the host wrapper), and
// this path serves callers that cannot use a second stream.
struct AgUnits {
  int unit_bytes, units_per_block;
};
__host__ __device__ __forceinline__ AgUnits ag_units(int K, int grid) {
  AgUnits u;
  u.unit_bytes = K * 2;
  u.units_per_block = BM;
  while (u.units_per_block < grid && u.unit_bytes >= 4096) {  // halves stay multiples of 16 bytes (K is a multiple of 64)
    u.unit_bytes >>= 1;
    u.units_per_block <<= 1;
  }
  return u;
}
__device__ void ag_send_units(const FusedParams& p, int at /*0..63*/, volatile int* abort_flag) {
  (void)abort_flag;  // nothing here waits for a peer, and both warps must reach every barrier: no early exit
  const int tmr = (p.M / p.npes) / BM;
  const AgUnits u = ag_units(p.K, (int)gridDim.x);
  const size_t block_bytes = (size_t)BM * p.K * 2;
  const int n16 = u.unit_bytes / 16;
  constexpr int UNROLL = 8;
  for (int o = 1; o < p.npes; ++o) {
    const int peer = (p.rank + o) % p.npes;
    for (int blk = 0; blk < tmr; ++blk) {
      for (int unit = (int)blockIdx.x; unit < u.units_per_block; unit += (int)gridDim.x) {
        const size_t off = (size_t)blk * block_bytes + (size_t)unit * u.unit_bytes;
        const uint4* src = (const uint4*)(p.ag_src + off);
        uint4* dst = (uint4*)(p.ag_dst[peer] + off);
        int i = at;
        for (; i + (UNROLL - 1) * AUX_THREADS < n16; i += UNROLL * AUX_THREADS) {
          uint4 v[UNROLL];
#pragma unroll
          for (int k = 0; k < UNROLL; ++k) v[k] = __ldg(src + i + k * AUX_THREADS);
#pragma unroll
          for (int k = 0; k < UNROLL; ++k) dst[i + k * AUX_THREADS] = v[k];
        }
        for (; i < n16; i += AUX_THREADS) dst[i] = __ldg(src + i);
      }
    }
    // The stores of all 64 threads are ordered before thread 0's release by the barrier (cumulativity).
    aux_bar_sync();
    if (at == 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      // units of a block that this CTA delivered: blockIdx.x, blockIdx.x + grid, … below units_per_block
      const int sent = (int)blockIdx.x < u.units_per_block ? (u.units_per_block - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      for (int blk = 0; blk < tmr && sent; ++blk) {
        uint64_t* f = p.ag_flags_peer[peer] + (size_t)p.rank * tmr + blk;
        asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(f), "l"((uint64_t)sent) : "memory");
      }
    }
  }
}

// MODE_RS / MODE_AR, switch path: reduction of the tiles this PE owns.  Work items are RED_ROWS-row slices (16 or 32) of the
// owned tiles, numbered in the order the tiles are produced and dealt round-robin to all auxiliary warps of the grid.
// A warp waits until all PEs have flagged the tile, then fetches each row slice with one `multimem.ld_reduce` per lane
// (a warp covers one 512-byte row of the tile per instruction): the switch adds the PEs' copies in fp32 and returns one
// bf16 result, so the owner receives one tile instead of npes - 1 partials and adds nothing itself.
//   RS: the sum is written to this PE's output.   AR: it is written once through the multicast alias of the output.
template <int RED_ROWS>
__device__ void switch_reduce(const FusedParams& p, int aw /*0..1*/, int lane, volatile int* abort_flag) {
  const int tiles_n = p.N / BN, tmr = (p.M / p.npes) / BM, per_peer = tmr * tiles_n;
  constexpr int GROUPS = BM / RED_ROWS;
  const int items = per_peer * GROUPS;
  const int nwarps = (int)gridDim.x * 2;
  const size_t pitch = (size_t)p.N * 2;
  for (int item = (int)blockIdx.x * 2 + aw; item < items; item += nwarps) {
    const int tile = item / GROUPS, g = item % GROUPS;
    const int n_tile = tile / tmr, m_local = tile % tmr;
    // Lane s watches PE s's flag of this tile; afterwards every lane performs an acquire of its own.
    uint32_t ok = 1;
    if (lane < p.npes) ok = wait_flag_ge(p.flags_local + (size_t)lane * per_peer + tile, p.epoch, p.wait_limit_ns, abort_flag) ? 1u : 0u;
    if (!__all_sync(0xffffffffu, ok)) return;
    {
      uint64_t v;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p.flags_local + (size_t)(lane % p.npes) * per_peer + tile) : "memory");
      (void)v;
    }
    const size_t row0 = (size_t)m_local * BM + (size_t)g * RED_ROWS;
    const size_t col_bytes = (size_t)n_tile * BN * 2 + (size_t)lane * 16;
    const char* src = p.stage_mc + ((size_t)p.rank * tmr * BM + row0) * pitch + col_bytes;
    uint4 v[RED_ROWS];
#pragma unroll
    for (int r = 0; r < RED_ROWS; ++r) v[r] = MultimemSum<__nv_bfloat16>::ld(src + (size_t)r * pitch);
    if (p.mode == BSHMEM_FUSED_AR) {
      char* dst = p.out_mc + ((size_t)p.rank * tmr * BM + row0) * pitch + col_bytes;
#pragma unroll
      for (int r = 0; r < RED_ROWS; ++r) multimem_st_v4(dst + (size_t)r * pitch, v[r]);
    } else {
      char* dst = p.out_local + row0 * pitch + col_bytes;
#pragma unroll
      for (int r = 0; r < RED_ROWS; ++r) *(uint4*)(dst + (size_t)r * pitch) = v[r];
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// Row-major bf16 matrix [rows, cols], box [box_rows, 64 columns], 128-byte swizzle.
static inline int make_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return BSHMEM_FUSED_ERR_DRIVER;
  if (((uintptr_t)base & 15) || (cols * 2) % 16) return BSHMEM_FUSED_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : BSHMEM_FUSED_ERR_DRIVER;
}


}  // namespace bshmem
