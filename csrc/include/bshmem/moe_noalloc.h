// An entry point for callers that are not allowed to allocate device memory.
// It has no counterpart in the reference library.
//
// Who needs it: code that runs where cudaMalloc (and every allocator built on
// it, torch's caching allocator included) is off limits -- a plug-in loaded into
// a serving process whose memory is fully budgeted by its host, a step running
// under a memory-accounting sandbox, or a latency-critical path where an
// allocation could stall behind another thread's free.  Such a caller can hand
// over its own input and output buffers but has nowhere to get the small
// scratch block (counters and a barrier word) that the MoE dispatch kernel
// needs.  Here that block lives inside the library, in a fixed array in device
// memory that exists from the moment the library is loaded on a GPU until the
// process ends.
//
// What it does: the single-PE form of the MoE dispatch -- all experts are local,
// so the kernel regroups the (token, expert) pairs by expert: for token t and
// slot j with expert id e, row x[t] is copied to a row inside expert e's segment
// of `recv_x`; `slot_map[t*K+j]` receives that row number and `expert_offsets`
// the segment boundaries.  Results match bshmem_moe_dispatch() with npes == 1
// (the order of rows inside a segment is not fixed in either).
//
// Limits and rules:
//   * experts <= BSHMEM_MOE_NOALLOC_MAX_EXPERTS (1024), top-k <= 16, H a multiple of 128;
//     anything beyond is refused with BSHMEM_MOE_ERR_SHAPE and a message on stderr.
//   * `recv_x` must hold T*K rows of H bf16 values.
//   * The built-in scratch is about 13 KB per GPU (BSHMEM_MOE_NOALLOC_SCRATCH_BYTES).
//   * The first call on a GPU looks up the array's device address; make that first call
//     outside any CUDA stream capture, with the GPU current.
//   * Every call on a GPU shares the one array: calls whose kernels could overlap on the
//     GPU (different streams, no ordering between them) race.  Issue them on one stream
//     or order them yourself.  Each call clears the words that must start at zero.
//   * Errors that the kernel meets (BSHMEM_MOE_ERRBIT_*) go to the caller's `error_flag`.  A caller that passes
//     none does not lose them: they go to a word inside the built-in array, which
//     bshmem_moe_noalloc_error_bits() reads back (it waits for the stream first).  The next call on the
//     same GPU clears that word, so read it before calling again.
//   * T * K must fit a 32-bit row number; larger products are refused with BSHMEM_MOE_ERR_SHAPE.
//   * No cudaMalloc, cudaFree or allocating library routine is called on this path.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#include "moe.h"

#ifdef __cplusplus
extern "C" {
#endif

#define BSHMEM_MOE_NOALLOC_MAX_EXPERTS 1024
#define BSHMEM_MOE_NOALLOC_SCRATCH_BYTES 13312

/* x: [T, H] bf16; topk_idx: [T, K] int32 (negative = skip); recv_x: [T*K, H] bf16 (out);
 * slot_map: [T, K] int32 (out); expert_offsets: [E + 1] int32 (out); error_flag: optional device
 * int that receives BSHMEM_MOE_ERRBIT_* bits (may be null).  Returns a BSHMEM_MOE_* status. */
int bshmem_moe_dispatch_local_noalloc(const void* x, const int* topk_idx, int T, int H, int K, int E, void* recv_x, int* slot_map, int* expert_offsets,
                                      int* error_flag, cudaStream_t stream);


/* For callers that passed no error_flag: waits for `stream`, then copies the error bits that the last call on
 * the current GPU recorded in the built-in array to *bits (host memory).  Allocates nothing. */
int bshmem_moe_noalloc_error_bits(cudaStream_t stream, int* bits);

#ifdef __cplusplus
}
#endif
