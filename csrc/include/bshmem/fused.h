// C interface of the fused GEMM + collective kernels (libbshmem_fused.so).
// The library is self-contained: it takes raw device pointers (local ones and,
// for the collective modes, the peers' mapped addresses of the same symmetric
// buffers) and a stream, and allocates nothing.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSHMEM_FUSED_MAX_PES 8

enum { BSHMEM_FUSED_PLAIN = 0, BSHMEM_FUSED_RS = 1, BSHMEM_FUSED_AR = 2, BSHMEM_FUSED_AG = 3, BSHMEM_FUSED_GROUPED = 4 };
#define BSHMEM_FUSED_MAX_GROUPS 256
/* SWIGLU (GROUPED only): every 64 output columns are 32 gate columns followed by their 32 up columns (the caller orders
 * the rows of B that way); the kernel writes silu(gate) * up, so `out` has N / 2 columns. */
enum { BSHMEM_FUSED_ACT_NONE = 0, BSHMEM_FUSED_ACT_GELU_TANH = 1, BSHMEM_FUSED_ACT_SWIGLU = 2 };
enum {
  BSHMEM_FUSED_OK = 0,
  BSHMEM_FUSED_ERR_ARGS = 1,
  BSHMEM_FUSED_ERR_SHAPE = 2,      /* M % (128*npes), N % 256 or K % 64 is not zero */
  BSHMEM_FUSED_ERR_ALIGNMENT = 3,  /* a base address or row pitch is not 16-byte aligned */
  BSHMEM_FUSED_ERR_DRIVER = 4
};

typedef struct {
  /* C[M,N] = A[M,K] * B[N,K]^T, all bf16 row-major.
   * PLAIN: A, B, out local.
   * RS   : every PE holds a K-slice; out is this PE's [M/npes, N] block of the sum over PEs.
   * AR   : as RS, but out is the full [M, N] sum on every PE (out_peer[] = each PE's out).
   * GROUPED: one PE; the rows of A fall into `groups` consecutive groups with boundaries group_offsets[0..groups] (a
   *        device array, read by the kernel: no host synchronisation), B holds one [N, K] matrix per group back to
   *        back, and rows r of group g give out[r, :] = A[r, :] * B_g^T.  M is the number of rows A and out are
   *        allocated for (any positive number); rows at or beyond group_offsets[groups] are not written.
   * AG   : A is this PE's gathered [M, K] buffer (symmetric); rows [rank*M/npes, …) hold this PE's shard on
   *        entry and the kernel fills the peers' copies (ag_peer[] = each PE's gathered buffer). */
  const void* A;
  const void* B;
  void* out;
  int M, N, K;
  int rank, npes, mode;
  uint64_t epoch;            /* call counter of this buffer set, starting at 1, identical on all PEs */
  uint32_t wait_limit_ms;    /* bound of every in-kernel wait; 0 = 10 s */
  int max_ctas;              /* 0 = one per SM */
  int n_comm;                /* unused (kept for layout compatibility): no CTA is set aside for sending */
  int* error_flag;           /* device int, OR-ed with 1 when a CTA gave up on a bounded wait */
  /* RS / AR */
  void* recv_local;                           /* push path: [npes][M/npes][N] bf16 receive slots (pick the half of this call's parity) */
  void* recv_peer[BSHMEM_FUSED_MAX_PES];      /* the same buffer on each PE */
  uint64_t* flags_local;                      /* [npes][(M/npes/128)*(N/256)] */
  uint64_t* flags_peer[BSHMEM_FUSED_MAX_PES];
  void* out_peer[BSHMEM_FUSED_MAX_PES];       /* AR only */
  /* AG */
  void* ag_peer[BSHMEM_FUSED_MAX_PES];
  uint64_t* ag_flags_local;                   /* [npes][M/npes/128] arrival counters (rows landed; 128 per call and block) */
  uint64_t* ag_flags_peer[BSHMEM_FUSED_MAX_PES];
  /* AR, optional: NVLink-multicast alias of `out` (nvshmemx_mc_ptr).  When set, a reduced tile leaves this GPU
   * once and the switch delivers it to every PE; when null it is stored to each PE's out in turn. */
  void* out_mc;
  /* RS / AR, optional: switch path.  stage_local is this PE's [M][N] bf16 staging buffer in symmetric memory (pick
   * the half of this call's parity), stage_mc its NVLink-multicast alias.  When both are set (and, for AR, out_mc),
   * partial tiles stay in the producing GPU's memory and the owner of a tile reads their sum with multimem.ld_reduce;
   * recv_local / recv_peer / out_peer are then unused. */
  void* stage_local;
  void* stage_mc;
  /* Activation applied to the fp32 result before it is rounded to bf16 (BSHMEM_FUSED_ACT_*); PLAIN and AG only
   * (a partial sum of RS / AR cannot be activated). */
  int act;
  /* AG: 1 = the caller pushes the shards itself (for example with copy engines on another stream) and sets
   * ag_flags[rank * (M/npes/128)] on each peer to `epoch` once its shard is complete there; the kernel then sends
   * nothing and waits for one flag per shard.  0 = two warps of every CTA send the shard. */
  int ag_external;
  /* GROUPED */
  const int* group_offsets;  /* device int32 [groups + 1], non-decreasing, group_offsets[groups] <= M */
  int groups;                /* 1 .. BSHMEM_FUSED_MAX_GROUPS */
} bshmem_fused_args_t;

/* Launches the kernel on `stream`.  Returns a BSHMEM_FUSED_* code. */
int bshmem_fused_gemm(const bshmem_fused_args_t* args, cudaStream_t stream);
int bshmem_fused_gemm_smem_bytes(void);

#ifdef __cplusplus
}
#endif
