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
constexpr int COMM_PIECE = 16384, COMM_BUFS = 8, COMM_AHEAD = 4;
constexpr int SMEM_TILES = 4 * (A_STAGE + BN * BK * 2) + EPI_BUFS * EPI_BUF;  // 4 stages of a 128 x 256 tile = 6 stages of a pair's halves
constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 256 /*barriers*/;
static_assert(COMM_PIECE * COMM_BUFS <= SMEM_TILES, "the sender's ring must fit in the GEMM's shared memory");

struct alignas(64) FusedParams {
  CUtensorMap tmA, tmB;
  CUtensorMap tmOut[BSHMEM_FUSED_MAX_PES];   // PLAIN/RS/AG: [0] is the local output; AR: output of each PE
  CUtensorMap tmRecv[BSHMEM_FUSED_MAX_PES];  // RS/AR: my slot in the receive buffer of each PE
  const __nv_bfloat16* recv_local;           // [npes][M/npes][N] partials received from each PE
  uint64_t* flags_local;                     // [npes][tiles per PE]
  uint64_t* flags_peer[BSHMEM_FUSED_MAX_PES];
  const char* ag_src;                        // my shard inside my gathered buffer
  char* ag_dst[BSHMEM_FUSED_MAX_PES];        // the same shard inside each PE's gathered buffer
  uint64_t* ag_flags_local;                  // [npes][m-tiles per shard]
  uint64_t* ag_flags_peer[BSHMEM_FUSED_MAX_PES];
  char* out_mc;                              // AR: multicast alias of the output (null: per-PE stores)
  int* error_flag;
  uint64_t epoch, wait_limit_ns, ag_unit_bytes;
  uint32_t ag_piece_bytes;  // size of one bulk copy of the sender (16-byte multiple, at most COMM_PIECE)
  int M, N, K, rank, npes, mode, n_comm, ag_parts, ag_tiles_per_unit;
};

struct TileInfo {
  int m_tile, n_tile;   // position in the full output
  int peer;             // RS/AR: PE that owns the rows; AG: PE whose shard holds the rows
  int m_local;          // m-tile index inside that PE's block of rows
  int idx_in_peer;      // tile number inside the block (flag index)
};

// Tile order.  Blocks of rows are visited peer by peer (RS/AR: rank+1, rank+2, …, own last; AG: own, rank-1, …);
// inside a block m runs fastest so that concurrently running CTAs share B tiles through L2.
__host__ __device__ __forceinline__ TileInfo tile_info(const FusedParams& p, int t) {
  const int tiles_n = p.N / BN;
  const int tmr = (p.M / p.npes) / BM;
  const int per_peer = tmr * tiles_n;
  const int o = t / per_peer, within = t % per_peer;
  TileInfo ti;
  if (p.mode == BSHMEM_FUSED_AG) ti.peer = (p.rank - o + p.npes) % p.npes;
  else ti.peer = (p.rank + 1 + o) % p.npes;
  ti.m_local = within % tmr;
  ti.n_tile = within / tmr;
  ti.m_tile = ti.peer * tmr + ti.m_local;
  ti.idx_in_peer = within;
  return ti;
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

// ------------------------------------------------------------------ all-gather sender (MODE_AG, extra CTAs)
__device__ void ag_sender(const FusedParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  if (threadIdx.x != 0) return;
  const int unit = blockIdx.x;  // one unit of my shard per sender CTA
  const size_t unit_off = (size_t)unit * p.ag_unit_bytes;
  const uint32_t PIECE = p.ag_piece_bytes;
  const int pieces = (int)(p.ag_unit_bytes / PIECE);
  const int tmr = (p.M / p.npes) / BM;
  uint32_t phase_bits = 0;  // one parity bit per ring slot
  for (int o = 1; o < p.npes && !*abort_flag; ++o) {
    const int peer = (p.rank + o) % p.npes;
    const char* src = p.ag_src + unit_off;
    char* dst = p.ag_dst[peer] + unit_off;
    const int ahead = pieces < COMM_AHEAD ? pieces : COMM_AHEAD;
    for (int q = 0; q < ahead; ++q) {
      mbar_expect_tx(&bars[q % COMM_BUFS], PIECE);
      bulk_load(smem + (q % COMM_BUFS) * COMM_PIECE, src + (size_t)q * PIECE, PIECE, &bars[q % COMM_BUFS]);
    }
    for (int q = 0; q < pieces; ++q) {
      const int nxt = q + COMM_AHEAD;
      if (nxt < pieces) {
        // Ring slot of piece `nxt` was last used by piece nxt-COMM_BUFS, stored COMM_BUFS-COMM_AHEAD iterations ago.
        bulk_wait_read<COMM_BUFS - COMM_AHEAD - 1>();
        mbar_expect_tx(&bars[nxt % COMM_BUFS], PIECE);
        bulk_load(smem + (nxt % COMM_BUFS) * COMM_PIECE, src + (size_t)nxt * PIECE, PIECE, &bars[nxt % COMM_BUFS]);
      }
      const int slot = q % COMM_BUFS;
      if (!mbar_wait(&bars[slot], (phase_bits >> slot) & 1, p.wait_limit_ns, abort_flag)) break;
      phase_bits ^= 1u << slot;
      bulk_store(dst + (size_t)q * PIECE, smem + slot * COMM_PIECE, PIECE);
      bulk_commit();
    }
    bulk_wait<0>();  // every byte of the unit has been written to the peer
    fence_proxy_async_all();
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    // Tell the peer which 128-row blocks are (partly) complete.
    const int first_tile = p.ag_parts > 1 ? unit / p.ag_parts : unit * p.ag_tiles_per_unit;
    const int ntiles = p.ag_parts > 1 ? 1 : p.ag_tiles_per_unit;
    for (int j = 0; j < ntiles; ++j) {
      uint64_t* f = p.ag_flags_peer[peer] + (size_t)p.rank * tmr + first_tile + j;
      asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(f), "l"((uint64_t)1) : "memory");
    }
  }
  bulk_wait<0>();
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
