// Fused tensor-parallel GEMM + collective for sm_100a, hand-written on
// tcgen05 / tensor memory / TMA.
//
//   C[M,N] = A[M,K] · B[N,K]^T      A, B, C bf16 (both operands K-major), fp32 accumulation in TMEM
//
// One persistent CTA per SM, 256 threads, warp-specialised:
//   warp 0    TMA producer   4-stage ring of {A 128x64, B 256x64} tiles (128-byte swizzle)
//   warp 1    MMA issuer     one thread issues tcgen05.mma 128x256x16, accumulators double-buffered in TMEM (2 x 256 columns)
//   warp 2    TMEM allocator, then auxiliary (with warp 3): the collective's data movement, see below
//   warps 4-7 epilogue       tcgen05.ld -> fp32 registers -> (+ peers' partial tiles) -> bf16 -> swizzled smem -> TMA store
// and the collective runs inside the same kernel, tile by tile, over peer memory:
//   MODE_RS  row-parallel GEMM -> reduce-scatter, two paths.
//            Switch path (the staging buffer has an NVLink-multicast alias): every PE walks the tiles in the same
//            order, TMA-stores each bf16 partial tile into its OWN staging buffer and flags the tile's owner; the
//            owner's auxiliary warps fetch the sum of all PEs' copies with `multimem.ld_reduce` (added inside the
//            switch) and write the output.  The epilogue never waits for a peer and never adds partials, the owner
//            receives one tile instead of npes - 1, and the reduction of a tile overlaps the main loops of later tiles.
//            Push path (no multicast): tiles whose rows belong to another PE are computed first (nearest destination
//            first) and TMA-stored as bf16 partials straight into that PE's receive slot, followed by a release flag
//            per tile.  The PE's own rows come last: their epilogue waits for the flags of the tile and adds the
//            partials to the TMEM accumulator before the single rounding to bf16.
//   MODE_AR  same; the reduced tile goes to every PE's output (one `multimem.st` through the switch, or per-PE stores).
//   MODE_AG  all-gather -> column-parallel GEMM.  This PE's activation shard is pushed into every peer's gathered
//            buffer, nearest peer first, either by copy engines on a second stream (the caller issues the copies and
//            a flag write per shard; no SM takes part) or by the auxiliary warps of all CTAs (a counter per 128-row
//            block); the producer warp consumes shards in arrival order (own, then rank-1, rank-2, …) and only waits
//            when one has not landed.  Remote data is always read from this GPU's own memory.
//   MODE_PLAIN  no collective (also what 1 PE runs).
// Every wait (mbarrier, flag) is bounded; on expiry the CTA unwinds, frees its tensor memory and sets `error_flag`.
// No load uses a cluster-wide broadcast form, so the same binary runs on any number of GPUs.
// (reference for the capability: examples/gemm_allreduce/*, which fuses a CUTLASS GEMM with an NVLS allreduce)
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <tuple>


#include "gemm_fused_common.cuh"

namespace bshmem {
using namespace sm100;

// ------------------------------------------------------------------ the kernel
// PAIR = false: every CTA owns 128 x 256 output tiles (4 stages of A 16 KB + B 32 KB).
// PAIR = true:  clusters of two CTAs; CTA r of a pair owns tile 2u + r of the same tile order, so the
// two tiles share their 256 columns.  Each CTA loads its own 128 rows of A and HALF of the B tile
// (6 stages of 16 KB + 16 KB), the even CTA issues one 256 x 256 x 16 MMA per K step for both, and each
// CTA's tensor memory receives its own 128 x 256 accumulator: per SM, half the B traffic from L2 and
// half the shared-memory reads per FLOP.  Everything after the accumulator (epilogue, flags, stores)
// is per CTA and identical in both variants.
template <bool PAIR>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_fused_kernel(const __grid_constant__ FusedParams p) {
  constexpr int STAGES = PAIR ? 6 : 4;
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  constexpr int B_STAGE = B_ROWS * BK * 2;
  static_assert(STAGES * (A_STAGE + B_STAGE) + EPI_BUFS * EPI_BUF == SMEM_TILES, "both variants use the same shared-memory budget");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE;
  uint8_t* sE = sB + STAGES * B_STAGE;
  uint64_t* bars = (uint64_t*)(smem + SMEM_TILES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* g_prefix = (int*)(smem + SMEM_TILES + 256);  // GROUPED: [groups + 1] tiles before each group

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], PAIR ? 2 : 1);  // pair: one arrival (with its byte count) from each CTA's producer
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], (PAIR ? 2 : 1) * (EPI_THREADS / 32));  // one arrival per epilogue warp
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  // Every tcgen05 instruction of a kernel carries the same .cta_group: the pair kernel allocates (and later frees)
  // tensor memory with cta_group::2, one warp of each CTA of the pair taking part.
  if (warp == 2) {
    tmem_alloc<PAIR ? 2 : 1>(tmem_slot, TMEM_COLS);
    tmem_relinquish<PAIR ? 2 : 1>();
  }
  const bool grouped = p.mode == BSHMEM_FUSED_GROUPED;
  if (grouped && warp == 3 && lane == 0) {
    // Tiles per group from the group boundaries in device memory: no host round trip decides the work list.
    int acc = 0;
    for (int g = 0; g < p.groups; ++g) {
      g_prefix[g] = acc;
      const int rows = p.group_offsets[g + 1] - p.group_offsets[g];
      acc += ((rows > 0 ? rows : 0) + BM - 1) / BM * (p.group_n / BN);
    }
    g_prefix[p.groups] = acc;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_n = p.N / BN;
  const int total_tiles = grouped ? g_prefix[p.groups] : (p.M / BM) * tiles_n;
  const int kblocks = p.K / BK;
  // Pair: worker u = pair index takes tiles 2u + r, 2(u + workers) + r, …
  const int first = PAIR ? ((int)blockIdx.x & ~1) + (int)cta_rank : (int)blockIdx.x;
  const int step = (int)gridDim.x;
  const int tmr = (p.M / p.npes) / BM;
  const bool reduce_mode = (p.mode == BSHMEM_FUSED_RS || p.mode == BSHMEM_FUSED_AR) && p.npes > 1;

  if (warp == 0) {
    // ---------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = first; t < total_tiles && !*abort_flag; t += step) {
        const TileInfo ti = grouped ? grouped_tile_info(p, g_prefix, t) : tile_info(p, t);
        if (p.mode == BSHMEM_FUSED_AG && ti.peer != p.rank) {
          // The 128 rows of this tile arrive from `peer`; all of K comes with them.
          // In-kernel sender: a counter per 128-row block.  External sender: one flag per shard, set to the call number.
          const uint64_t want = p.ag_external ? p.epoch : p.epoch * (uint64_t)ag_units(p.K, (int)gridDim.x).units_per_block;
          const size_t fidx = (size_t)ti.peer * tmr + (p.ag_external ? 0 : ti.m_local);
          if (!wait_flag_ge(p.ag_flags_local + fidx, want, p.wait_limit_ns, abort_flag)) break;
          fence_proxy_async_all();  // peer-written data (generic proxy) before my TMA reads (async proxy)
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, p.wait_limit_ns, abort_flag)) break;
          if (PAIR) {
            const uint32_t lead = mapa_u32(smem_u32(&full[stage]), 0);
            mbar_expect_tx_cluster(lead, A_STAGE + B_STAGE);
            tma_load_2d_pair(sA + stage * A_STAGE, &p.tmA, lead, kb * BK, ti.a_row);
            tma_load_2d_pair(sB + stage * B_STAGE, &p.tmB, lead, kb * BK, ti.b_row + (int)cta_rank * B_ROWS);
          } else {
            mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
            tma_load_2d(sA + stage * A_STAGE, &p.tmA, &full[stage], kb * BK, ti.a_row);
            tma_load_2d(sB + stage * B_STAGE, &p.tmB, &full[stage], kb * BK, ti.b_row);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // The MMA side still arrives on the empty barriers of the last fills: wait for those arrivals,
      // so that none of them (in a pair they come from the other SM) finds this CTA gone.
      for (int i = 0; i < STAGES && !*abort_flag; ++i) {
        if (!mbar_wait(&empty[stage], phase ^ 1, p.wait_limit_ns, abort_flag)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if ((!PAIR || cta_rank == 0) && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(PAIR ? 2 * BM : BM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int t = first; t < total_tiles && !*abort_flag; t += step) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.wait_limit_ns, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * ACC_COLS);
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.wait_limit_ns, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = umma_desc_k_sw128(smem_u32(sA + stage * A_STAGE));
          const uint64_t db = umma_desc_k_sw128(smem_u32(sB + stage * B_STAGE));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // Advancing K inside the 128-byte swizzle atom: +32 bytes = +2 in descriptor address units.
            if (PAIR) umma_bf16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
            else umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          }
          // The stage is free (in both CTAs of a pair) once these MMAs have read it.
          if (PAIR) umma_commit_pair(&empty[stage]);
          else umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) umma_commit_pair(&acc_full[acc]);
        else umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < EPI_WARP0) {
    // ---------------- auxiliary warps 2 and 3
    if (p.mode == BSHMEM_FUSED_AG && p.npes > 1 && !p.ag_external) ag_send_units(p, (int)threadIdx.x - AUX_WARP0 * 32, abort_flag);
    else if (reduce_mode && p.sw_reduce && p.red_rows == 32) switch_reduce<32>(p, warp - AUX_WARP0, lane, abort_flag);
    else if (reduce_mode && p.sw_reduce) switch_reduce<16>(p, warp - AUX_WARP0, lane, abort_flag);
  } else {
    // ---------------- epilogue
    const int ew = warp - EPI_WARP0;                 // TMEM lane quarter of this warp
    const int row = ew * 32 + lane;                  // row of the tile handled by this thread
    const bool issuer = threadIdx.x == EPI_WARP0 * 32;
    const bool sw = reduce_mode && p.sw_reduce;  // every tile goes to the local staging buffer; the auxiliary warps reduce
    int acc = 0;
    uint32_t acc_phase = 0, chunk_counter = 0;
    uint64_t* pending_flag = nullptr;  // flag of the previous remote tile, published once its stores have completed
    for (int t = first; t < total_tiles; t += step) {
      const TileInfo ti = grouped ? grouped_tile_info(p, g_prefix, t) : tile_info(p, t);
      const bool own = !reduce_mode || (!sw && ti.peer == p.rank);
      uint32_t ok = mbar_wait(&acc_full[acc], acc_phase, p.wait_limit_ns, abort_flag) ? 1u : 0u;
      if (issuer && pending_flag) {
        // The previous tile's stores were issued a whole main loop ago: this wait does not stall.
        bulk_wait<0>();
        fence_proxy_async_all();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(pending_flag), "l"(p.epoch) : "memory");
        pending_flag = nullptr;
      }
      if (reduce_mode && own && issuer && ok) {
        // Partials of this tile from every other PE must have landed in my receive slots.
        for (int s = 0; s < p.npes && ok; ++s)
          if (s != p.rank && !wait_flag_ge(p.flags_local + (size_t)s * (tmr * tiles_n) + ti.idx_in_peer, p.epoch, p.wait_limit_ns, abort_flag)) ok = 0;
      }
      // One vote per tile keeps the 128 epilogue threads together: either all go on or all leave.
      if (!named_bar_and(1, EPI_THREADS, ok)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * ACC_COLS);
#pragma unroll 1
      for (int c = 0; c < BN / EPI_COLS; ++c) {
        float f[EPI_COLS];
        tmem_ld_32x32(t_row + c * EPI_COLS, (uint32_t*)f);
        tmem_ld_32x32(t_row + c * EPI_COLS + 32, (uint32_t*)f + 32);
        tmem_ld_wait();
        if (c == BN / EPI_COLS - 1) {
          // All of this accumulator is in registers: hand the TMEM buffer back to the MMA warp.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[acc]), 0));
            else mbar_arrive(&acc_empty[acc]);
          }
        }
        if (p.act == BSHMEM_FUSED_ACT_GELU_TANH) {
          // tanh-approximated GELU on the fp32 accumulators, before the single rounding to bf16.
#pragma unroll
          for (int j = 0; j < EPI_COLS; ++j) f[j] = gelu_tanh(f[j]);
        }
        if (reduce_mode && own) {
          const size_t rows_per_pe = (size_t)p.M / p.npes;
          const size_t grow = (size_t)ti.m_local * BM + row;
          const size_t col0 = (size_t)ti.n_tile * BN + (size_t)c * EPI_COLS;
          // Partials of two senders are loaded (16 x 16 bytes per thread in flight) before either is added:
          // the epilogue of an own tile reads (npes - 1) x 64 KB and must not outlast the next tile's main loop.
          auto add8 = [&](const uint4* v) {
#pragma unroll
            for (int j = 0; j < EPI_COLS / 8; ++j) {
              const __nv_bfloat162* h = (const __nv_bfloat162*)&v[j];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 x = __bfloat1622float2(h[e]);
                f[j * 8 + 2 * e] += x.x;
                f[j * 8 + 2 * e + 1] += x.y;
              }
            }
          };
          for (int q = 0; q < p.npes - 1; q += 2) {
            const bool two = q + 1 < p.npes - 1;
            const int s0 = (p.rank + 1 + q) % p.npes, s1 = (p.rank + 2 + q) % p.npes;
            const uint4* a0 = (const uint4*)(p.recv_local + ((size_t)s0 * rows_per_pe + grow) * p.N + col0);
            const uint4* a1 = (const uint4*)(p.recv_local + ((size_t)s1 * rows_per_pe + grow) * p.N + col0);
            uint4 v0[EPI_COLS / 8], v1[EPI_COLS / 8];
#pragma unroll
            for (int j = 0; j < EPI_COLS / 8; ++j) v0[j] = a0[j];
            if (two) {
#pragma unroll
              for (int j = 0; j < EPI_COLS / 8; ++j) v1[j] = a1[j];
            }
            add8(v0);
            if (two) add8(v1);
          }
        }
        if (grouped) {
          // Ragged tiles: every thread writes its own row straight from registers (128 contiguous bytes per chunk),
          // rows past the end of the group are dropped.  No shared-memory staging, no bulk store.
          if (p.act == BSHMEM_FUSED_ACT_SWIGLU) {
            // Gated activation: the 64 columns of a chunk are 32 gate columns followed by their 32 up columns (the
            // caller interleaves the weight rows that way); the output has half as many columns.
#pragma unroll
            for (int j = 0; j < EPI_COLS / 2; ++j) f[j] = f[j] / (1.0f + __expf(-f[j])) * f[EPI_COLS / 2 + j];
          }
          const int out_cols = p.act == BSHMEM_FUSED_ACT_SWIGLU ? EPI_COLS / 2 : EPI_COLS;
          const size_t pitch = p.act == BSHMEM_FUSED_ACT_SWIGLU ? (size_t)p.group_n / 2 : (size_t)p.group_n;
          if (row < ti.valid_rows) {
            uint4* o = (uint4*)(p.out_local + ((size_t)(ti.a_row + row) * pitch + ((size_t)ti.n_tile * (BN / EPI_COLS) + (size_t)c) * out_cols) * 2);
#pragma unroll
            for (int j = 0; j < EPI_COLS / 8; ++j) {
              if (j * 8 >= out_cols) break;
              uint4 v;
              __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
              for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[j * 8 + 2 * e], f[j * 8 + 2 * e + 1]);
              o[j] = v;
            }
          }
          continue;
        }
        // Staging buffer (chunk_counter & 1) must have been drained by the TMA store issued two chunks ago.
        uint8_t* buf = sE + (chunk_counter & 1) * EPI_BUF;
        if (issuer) bulk_wait_read<1>();
        named_bar_sync(1, EPI_THREADS);
        // Row `row` of the chunk is 128 bytes = 8 x 16-byte pieces; piece j goes to slot j ^ (row & 7) (128-byte swizzle).
#pragma unroll
        for (int j = 0; j < EPI_COLS / 8; ++j) {
          uint4 v;
          __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[j * 8 + 2 * e], f[j * 8 + 2 * e + 1]);
          *(uint4*)(buf + row * 128 + ((j ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (own && p.mode == BSHMEM_FUSED_AR && p.npes > 1 && p.out_mc) {
          // Reduced tile of an all-reduce: every thread takes 16-byte pieces of the staged chunk, a warp
          // covering four whole 128-byte rows per store, and writes them through the multicast alias:
          // one copy leaves this GPU and the switch delivers it to all PEs (this one included).
          char* base = p.out_mc + ((size_t)ti.m_tile * BM * p.N + (size_t)ti.n_tile * BN + (size_t)c * EPI_COLS) * 2;
#pragma unroll
          for (int i = 0; i < EPI_COLS * 2 * BM / 16 / EPI_THREADS; ++i) {
            const int idx = i * EPI_THREADS + (int)threadIdx.x - EPI_WARP0 * 32;
            const int r = idx >> 3, j = idx & 7;
            const uint4 v = *(const uint4*)(buf + r * 128 + ((j ^ (r & 7)) << 4));
            multimem_st_v4(base + (size_t)r * p.N * 2 + j * 16, v);
          }
        } else if (issuer) {
          const int x = ti.n_tile * BN + c * EPI_COLS;
          if (sw) {
            tma_store_2d(&p.tmStage, buf, x, ti.m_tile * BM);
          } else if (!own) {
            tma_store_2d(&p.tmRecv[ti.peer], buf, x, ti.m_local * BM);
          } else if (p.mode == BSHMEM_FUSED_AR && p.npes > 1) {
            for (int q = 0; q < p.npes; ++q) tma_store_2d(&p.tmOut[(p.rank + q) % p.npes], buf, x, ti.m_tile * BM);
          } else if (p.mode == BSHMEM_FUSED_RS) {
            tma_store_2d(&p.tmOut[0], buf, x, ti.m_local * BM);
          } else {
            tma_store_2d(&p.tmOut[0], buf, x, ti.m_tile * BM);
          }
          bulk_commit();
        }
        ++chunk_counter;
      }
      // Waiting here for the remote writes would idle the epilogue for a link round trip per tile;
      // the flag goes out at the start of the next tile's epilogue instead (or after the loop).
      if (sw) {
        // The partial tile stays in this GPU's memory: its stores complete within a microsecond or two, and the
        // owner is told at once so that the reduction runs while the next tiles are computed.
        if (issuer) {
          bulk_wait<0>();
          fence_proxy_async_all();
          uint64_t* f = (ti.peer == p.rank ? p.flags_local : p.flags_peer[ti.peer]) + (size_t)p.rank * (tmr * tiles_n) + ti.idx_in_peer;
          asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f), "l"(p.epoch) : "memory");
        }
      } else if (!own && issuer) {
        pending_flag = p.flags_peer[ti.peer] + (size_t)p.rank * (tmr * tiles_n) + ti.idx_in_peer;
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) {
      bulk_wait<0>();
      if (pending_flag) {
        fence_proxy_async_all();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(pending_flag), "l"(p.epoch) : "memory");
      }
    }
  }

  // ---------------- teardown
  if (*abort_flag) {
    // Give copies that are still in flight time to land before the CTA's shared memory goes away.
    const uint64_t t0 = timer_ns();
    while (timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  // Pair: neither CTA leaves (or frees tensor memory the leader's MMAs write) before both are done.
  if (PAIR) cluster_sync_all();
  if (warp == 2) tmem_dealloc<PAIR ? 2 : 1>(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 1);
}

static int g_attr_set_for_device = -1;

// CTA pairs are the default where the shape allows them; BSHMEM_FUSED_2CTA=0 selects one CTA per tile.
static bool pair_wanted() {
  static const bool on = [] {
    const char* e = getenv("BSHMEM_FUSED_2CTA");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace bshmem

using namespace bshmem;

extern "C" int bshmem_fused_gemm(const bshmem_fused_args_t* a, cudaStream_t stream) {
  if (!a || !a->A || !a->B || !a->out || !a->error_flag) return BSHMEM_FUSED_ERR_ARGS;
  const int npes = a->npes, mode = a->mode;
  if (npes < 1 || npes > BSHMEM_FUSED_MAX_PES || a->rank < 0 || a->rank >= npes) return BSHMEM_FUSED_ERR_ARGS;
  const bool grouped = mode == BSHMEM_FUSED_GROUPED;
  if (grouped && (npes != 1 || !a->group_offsets || a->groups < 1 || a->groups > MAX_GROUPS)) return BSHMEM_FUSED_ERR_ARGS;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || (!grouped && a->M % (BM * npes)) || a->N % BN || a->K % BK) return BSHMEM_FUSED_ERR_SHAPE;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K; p.rank = a->rank; p.npes = npes; p.mode = mode;
  p.epoch = a->epoch;
  if (a->act != BSHMEM_FUSED_ACT_NONE && a->act != BSHMEM_FUSED_ACT_GELU_TANH && !(a->act == BSHMEM_FUSED_ACT_SWIGLU && mode == BSHMEM_FUSED_GROUPED)) return BSHMEM_FUSED_ERR_ARGS;
  if (a->act != BSHMEM_FUSED_ACT_NONE && (mode == BSHMEM_FUSED_RS || mode == BSHMEM_FUSED_AR) && npes > 1) return BSHMEM_FUSED_ERR_ARGS;  // partial sums
  p.act = a->act;
  p.wait_limit_ns = a->wait_limit_ms ? (uint64_t)a->wait_limit_ms * 1000000ull : 10000000000ull;
  p.error_flag = a->error_flag;
  const int rows_per_pe = a->M / npes;
  const int tmr = rows_per_pe / BM;
  int device = 0, sms = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  int grid = a->max_ctas > 0 && a->max_ctas < sms ? a->max_ctas : sms;
  // A pair takes two consecutive 128-row tiles of one PE's block of rows.
  bool pair = pair_wanted() && rows_per_pe % (2 * BM) == 0 && grid >= 2 && !grouped;  // ragged groups do not pair up
  if (pair) grid &= ~1;
  int st = make_map(&p.tmA, a->A, a->M, a->K, BM);
  if (st) return st;
  const bool reduce_mode = (mode == BSHMEM_FUSED_RS || mode == BSHMEM_FUSED_AR) && npes > 1;
  if (mode == BSHMEM_FUSED_AR && npes > 1) {
    p.out_mc = (char*)a->out_mc;
    const bool sw = a->stage_local && a->stage_mc && a->out_mc;  // the switch path stores through out_mc only
    for (int q = 0; q < npes && !st && !sw; ++q) {
      if (!a->out_peer[q]) return BSHMEM_FUSED_ERR_ARGS;
      st = make_map(&p.tmOut[q], a->out_peer[q], a->M, a->N, BM);
    }
  } else {
    st = make_map(&p.tmOut[0], a->out, mode == BSHMEM_FUSED_RS ? rows_per_pe : a->M, a->N, BM);
  }
  if (st) return st;
  if (reduce_mode) {
    if (!a->flags_local) return BSHMEM_FUSED_ERR_ARGS;
    p.flags_local = a->flags_local;
    // Switch path: a staging buffer with a multicast alias (and, for the all-reduce, a multicast alias of the output).
    p.sw_reduce = a->stage_local && a->stage_mc && (mode == BSHMEM_FUSED_RS || a->out_mc);
    if (p.sw_reduce) {
      static const int red_rows = [] {
        const char* e = getenv("BSHMEM_FUSED_RED_ROWS");
        return e && atoi(e) == 16 ? 16 : 32;
      }();
      p.red_rows = red_rows;
      if (((uintptr_t)a->stage_mc & 15) || ((uintptr_t)a->out & 15) || ((uintptr_t)a->out_mc & 15)) return BSHMEM_FUSED_ERR_ALIGNMENT;
      p.stage_mc = (const char*)a->stage_mc;
      p.out_local = (char*)a->out;
      st = make_map(&p.tmStage, a->stage_local, a->M, a->N, BM);
    } else {
      if (!a->recv_local) return BSHMEM_FUSED_ERR_ARGS;
      p.recv_local = (const __nv_bfloat16*)a->recv_local;
    }
    for (int q = 0; q < npes && !st; ++q) {
      if (q == a->rank) continue;
      if (!a->flags_peer[q] || (!p.sw_reduce && !a->recv_peer[q])) return BSHMEM_FUSED_ERR_ARGS;
      p.flags_peer[q] = a->flags_peer[q];
      if (p.sw_reduce) continue;
      // My slot (index `rank`) inside PE q's receive buffer.
      const char* slot = (const char*)a->recv_peer[q] + (size_t)a->rank * rows_per_pe * a->N * 2;
      st = make_map(&p.tmRecv[q], slot, rows_per_pe, a->N, BM);
    }
    if (st) return st;
  }
  if (mode == BSHMEM_FUSED_AG && npes > 1) {
    if (!a->ag_flags_local) return BSHMEM_FUSED_ERR_ARGS;
    const size_t shard_bytes = (size_t)rows_per_pe * a->K * 2;
    p.ag_src = (const char*)a->A + (size_t)a->rank * shard_bytes;
    p.ag_flags_local = a->ag_flags_local;
    for (int q = 0; q < npes; ++q) {
      if (q == a->rank) continue;
      if (!a->ag_peer[q] || !a->ag_flags_peer[q]) return BSHMEM_FUSED_ERR_ARGS;
      p.ag_dst[q] = (char*)a->ag_peer[q] + (size_t)a->rank * shard_bytes;
      p.ag_flags_peer[q] = a->ag_flags_peer[q];
    }
    p.ag_external = a->ag_external != 0;
  }
  if (grouped) {
    if ((uintptr_t)a->out & 15) return BSHMEM_FUSED_ERR_ALIGNMENT;
    p.group_offsets = a->group_offsets;
    p.groups = a->groups;
    p.group_n = a->N;
    p.out_local = (char*)a->out;
  }
  st = make_map(&p.tmB, a->B, grouped ? (uint64_t)a->groups * a->N : (uint64_t)a->N, a->K, pair ? BN / 2 : BN);
  if (st) return st;
  if (g_attr_set_for_device != device) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) {
      fprintf(stderr, "bshmem_fused_gemm: cannot reserve %d bytes of shared memory: %s\n", SMEM_BYTES, cudaGetErrorString(e));
      return BSHMEM_FUSED_ERR_DRIVER;
    }
    g_attr_set_for_device = device;
  }
  cudaError_t e;
  if (pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemm_fused_kernel<true>, p);
  } else {
    gemm_fused_kernel<false><<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    fprintf(stderr, "bshmem_fused_gemm: launch failed: %s\n", cudaGetErrorString(e));
    return BSHMEM_FUSED_ERR_DRIVER;
  }
  return 0;
}

extern "C" int bshmem_fused_gemm_smem_bytes(void) { return SMEM_BYTES; }

// Test hook (host only): how the all-gather mode cuts a 128-row block of a shard into units for `grid` CTAs.
// out = {unit_bytes, units_per_block}.
extern "C" int bshmem_fused_test_ag_units(int K, int grid, int* out) {
  if (K <= 0 || K % BK || grid <= 0) return 1;
  const AgUnits u = ag_units(K, grid);
  out[0] = u.unit_bytes;
  out[1] = u.units_per_block;
  return 0;
}

// Test hook (host only): the tile that position `t` of the tile order names, for the checks of the order's
// invariants (every tile once, own rows last, pairs share their columns).  out = {m_tile, n_tile, peer, m_local, idx_in_peer}.
// `mode` may carry 0x100 to ask for the order of the switch path of RS / AR.
extern "C" int bshmem_fused_test_tile_info(int mode, int M, int N, int rank, int npes, int t, int* out) {
  if (npes < 1 || M % (BM * npes) || N % BN || t < 0 || t >= (M / BM) * (N / BN)) return 1;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.sw_reduce = (mode & 0x100) != 0;
  mode &= 0xff;
  p.mode = mode; p.M = M; p.N = N; p.rank = rank; p.npes = npes;
  const TileInfo ti = tile_info(p, t);
  out[0] = ti.m_tile; out[1] = ti.n_tile; out[2] = ti.peer; out[3] = ti.m_local; out[4] = ti.idx_in_peer;
  return 0;
}
