// C interface of the expert-parallel dispatch / combine kernels (libbshmem_fused.so).
//
// dispatch: every PE holds T tokens of H bf16 values and, per token, K expert ids out of E
// (expert e lives on PE e / (E/npes)).  One cooperative kernel counts, exchanges the counts with
// all PEs, derives where each (token, expert) pair lands and pushes the rows straight into the
// receive buffer of the owning PE, grouped by expert, then by source PE.  The rows travel as bf16
// or as fp8 e4m3 with one fp32 scale per 128 values (quantised on the fly).
// combine: the inverse; every PE pulls, for each of its tokens, the K expert outputs from the PEs
// that own them and writes their weighted sum.
// The library allocates nothing: receive buffers, the count matrix and the flags are symmetric
// buffers supplied by the caller (the peers' mapped addresses of the same objects), the small
// scratch block is local device memory.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSHMEM_MOE_MAX_PES 8
#define BSHMEM_MOE_MAX_EXPERTS 1024
#define BSHMEM_MOE_MAX_TOPK 16
#define BSHMEM_MOE_QUANT_BLOCK 128

enum { BSHMEM_MOE_BF16 = 0, BSHMEM_MOE_FP8_E4M3 = 1 };
enum { BSHMEM_MOE_OK = 0, BSHMEM_MOE_ERR_ARGS = 1, BSHMEM_MOE_ERR_SHAPE = 2, BSHMEM_MOE_ERR_DRIVER = 3 };
/* bits OR-ed into *error_flag by the kernels */
#define BSHMEM_MOE_ERRBIT_TIMEOUT 1   /* a bounded wait (grid or cross-PE barrier) expired */
#define BSHMEM_MOE_ERRBIT_OVERFLOW 2  /* a receive buffer was too small; the rows beyond it were dropped */

typedef struct {
  int T, H, K, E, rank, npes;
  int payload;             /* BSHMEM_MOE_BF16 or BSHMEM_MOE_FP8_E4M3 */
  int cap_rows;            /* rows each PE's receive buffer can hold */
  uint64_t epoch;          /* call counter of this buffer set, starting at 1, identical on all PEs */
  uint32_t wait_limit_ms;  /* bound of every in-kernel wait; 0 = 10 s */
  int max_ctas;            /* 0 = as many as can be co-resident */
  int* error_flag;         /* device int */
  /* inputs (local) */
  const void* x;           /* [T, H] bf16 */
  const int* topk_idx;     /* [T, K] expert ids; a negative id drops that slot */
  /* outputs */
  void* recv_x[BSHMEM_MOE_MAX_PES];       /* every PE's receive buffer: [cap_rows, H] bf16 or [cap_rows, H] bytes */
  float* recv_scale[BSHMEM_MOE_MAX_PES];  /* fp8 only: [cap_rows, H/128] */
  int* slot_map;           /* [T, K] row taken in the owner's receive buffer (-1: dropped) */
  int* expert_offsets;     /* [E/npes + 1] first row of each local expert in MY receive buffer */
  int* src_offsets;        /* [E/npes, npes] first row of each (local expert, source PE) segment; may be null */
  /* symmetric helpers */
  int* counts[BSHMEM_MOE_MAX_PES];        /* [npes, E] int32 count matrix on every PE */
  uint64_t* flags[BSHMEM_MOE_MAX_PES];    /* [4, npes] uint64 barrier flags on every PE */
  /* local scratch: bshmem_moe_scratch_bytes(E) bytes, 256-byte aligned, contents irrelevant on entry */
  void* scratch;
  /* Optional: [cap_rows] int32 on every PE (symmetric).  When set, a token that goes to several experts of one PE
   * crosses NVLink once: its row is written to the first of its rows on that PE, the other rows receive only the
   * number of that first row here, and the receiving PE copies the row locally before the kernel ends.  Null on every
   * entry = every (token, expert) pair is sent (the only form with one PE). */
  int* dup_src[BSHMEM_MOE_MAX_PES];
} bshmem_moe_dispatch_args_t;

typedef struct {
  int T, H, K, E, rank, npes;
  uint64_t epoch;
  uint32_t wait_limit_ms;
  int max_ctas;
  int* error_flag;
  const void* y[BSHMEM_MOE_MAX_PES];      /* every PE's expert-output buffer: [cap_rows, H] bf16, same row numbering as recv_x */
  const int* topk_idx;     /* [T, K] */
  const float* topk_weight;/* [T, K] */
  const int* slot_map;     /* [T, K] from dispatch */
  void* out;               /* [T, H] bf16 */
  uint64_t* flags[BSHMEM_MOE_MAX_PES];    /* same flag block as dispatch (rows 2 and 3 are used here) */
  void* scratch;
} bshmem_moe_combine_args_t;

size_t bshmem_moe_scratch_bytes(int experts);
int bshmem_moe_dispatch(const bshmem_moe_dispatch_args_t* args, cudaStream_t stream);
int bshmem_moe_combine(const bshmem_moe_combine_args_t* args, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
