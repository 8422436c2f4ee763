// Launchers of the on-stream collectives and the single-thread helper kernels of
// the on-stream point-to-point API.  `dtype` is a bshmem::DType, `op` a
// bshmem::ReduceOp, `algo` 0 for the automatic choice.  All return a Status.
#pragma once
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace bshmem {

int coll_reduce_on_stream(int team, void* dst, const void* src, size_t n, int dtype, int op, cudaStream_t stream, int algo = 0);
int coll_reducescatter_on_stream(int team, void* dst, const void* src, size_t nreduce, int dtype, int op, cudaStream_t stream, int algo = 0);
int coll_fcollect_on_stream(int team, void* dst, const void* src, size_t block_bytes, cudaStream_t stream, int algo = 0);
int coll_alltoall_on_stream(int team, void* dst, const void* src, size_t block_bytes, cudaStream_t stream);
int coll_broadcast_on_stream(int team, void* dst, const void* src, size_t bytes, int root, cudaStream_t stream, int algo = 0);
int coll_maxloc_on_stream(int team, void* dst, const void* src, cudaStream_t stream);
int coll_barrier_on_stream(int team, cudaStream_t stream, bool with_quiet);

int p2p_wait_until_on_stream(const void* ivar, int cmp, uint64_t value, int width, bool is_signed, cudaStream_t stream);
int p2p_wait_until_all_on_stream(const uint64_t* ivars, size_t n, const int* status, int cmp, const uint64_t* values, uint64_t value, cudaStream_t stream);
int p2p_signal_op_on_stream(uint64_t* sig, uint64_t value, int op, int pe, cudaStream_t stream);
int p2p_quiet_on_stream(cudaStream_t stream);

}  // namespace bshmem
