// Host-side public API, source compatible with NVSHMEM's host headers: the
// OpenSHMEM-style nvshmem_* calls and the nvshmemx_* extensions (unique-id
// init, on-stream operations, teams, collective launch).  Typed families are
// expanded from the tables in bshmem/types.h
// (reference: src/include/host/nvshmem_api.h, nvshmemx_api.h, nvshmem_coll_api.h, nvshmemx_coll_api.h).
#pragma once
#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#include "bshmem/state.h"
#include "bshmem/types.h"

/* Calls that exist on both sides are declared __host__ __device__ under nvcc: the host
 * definition lives in the host library, the device definition in bshmem/device_api.cuh
 * (visible only to the device compilation pass). */
#ifdef __CUDACC__
#define BSHMEM_HD __host__ __device__
#else
#define BSHMEM_HD
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- constants */
#define NVSHMEM_MAJOR_VERSION 1
#define NVSHMEM_MINOR_VERSION 3
#define NVSHMEM_MAX_NAME_LEN 256
#define NVSHMEM_VENDOR_STRING BSHMEM_VENDOR_STRING
#define NVSHMEM_VENDOR_MAJOR_VERSION BSHMEM_MAJOR
#define NVSHMEM_VENDOR_MINOR_VERSION BSHMEM_MINOR
#define NVSHMEM_VENDOR_PATCH_VERSION BSHMEM_PATCH

enum nvshmemi_cmp_type { NVSHMEM_CMP_EQ = 0, NVSHMEM_CMP_NE, NVSHMEM_CMP_GT, NVSHMEM_CMP_LE, NVSHMEM_CMP_LT, NVSHMEM_CMP_GE, NVSHMEM_CMP_SENTINEL = 0x7fffffff };
enum nvshmemi_thread_support { NVSHMEM_THREAD_SINGLE = 0, NVSHMEM_THREAD_FUNNELED, NVSHMEM_THREAD_SERIALIZED, NVSHMEM_THREAD_MULTIPLE, NVSHMEM_THREAD_TYPE_SENTINEL = 0x7fffffff };
enum { NVSHMEM_STATUS_NOT_INITIALIZED = 0, NVSHMEM_STATUS_IS_BOOTSTRAPPED, NVSHMEM_STATUS_IS_INITIALIZED, NVSHMEM_STATUS_LIMITED_MPG, NVSHMEM_STATUS_FULL_MPG, NVSHMEM_STATUS_INVALID = 0x7fffffff };
enum nvshmemx_status {
  NVSHMEMX_SUCCESS = 0, NVSHMEMX_ERROR_INVALID_VALUE, NVSHMEMX_ERROR_OUT_OF_MEMORY, NVSHMEMX_ERROR_NOT_SUPPORTED,
  NVSHMEMX_ERROR_SYMMETRY, NVSHMEMX_ERROR_GPU_NOT_SELECTED, NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED, NVSHMEMX_ERROR_INTERNAL,
  NVSHMEMX_ERROR_SENTINEL = 0x7fffffff
};
#define NVSHMEM_SIGNAL_SET 9
#define NVSHMEM_SIGNAL_ADD 10
#define NVSHMEMX_PE_ANY (-1)

enum { NVSHMEMX_INIT_THREAD_PES = 1, NVSHMEMX_INIT_WITH_MPI_COMM = 1 << 1, NVSHMEMX_INIT_WITH_SHMEM = 1 << 2, NVSHMEMX_INIT_WITH_UNIQUEID = 1 << 3, NVSHMEMX_INIT_MAX = 1 << 31 };

typedef int32_t nvshmem_team_t;
typedef nvshmem_team_t nvshmemx_team_t;
#define NVSHMEM_TEAM_INVALID (-1)
#define NVSHMEM_TEAM_WORLD 0
#define NVSHMEM_TEAM_SHARED 1
#define NVSHMEMX_TEAM_NODE 2
#define NVSHMEMX_TEAM_SAME_MYPE_NODE 3
#define NVSHMEMI_TEAM_SAME_GPU 4
#define NVSHMEMI_TEAM_GPU_LEADERS 5
#define NVSHMEM_TEAM_NUM_CONTEXTS 1

/* ---------------------------------------------------------------- ABI structs (version = (ver << 16) + sizeof) */
typedef struct { int version; char internal[124]; } nvshmemx_uniqueid_t;
typedef struct { int version; nvshmemx_uniqueid_t* id; int myrank; int nranks; } nvshmemx_uniqueid_args_t;
typedef struct { int version; nvshmemx_uniqueid_args_t uid_args; int cuda_device_id; char content[92]; } nvshmemx_init_args_t;
typedef struct { int version; void* mpi_comm; nvshmemx_init_args_t args; } nvshmemx_init_attr_t;
typedef uint64_t nvshmemx_team_uniqueid_t;
typedef struct { int version; int num_contexts; nvshmemx_team_uniqueid_t uniqueid; char padding[48]; } nvshmem_team_config_t;
#ifdef __cplusplus
static_assert(sizeof(nvshmemx_uniqueid_t) == 128, "unique id is 128 bytes");
static_assert(sizeof(nvshmemx_uniqueid_args_t) == 24, "unique id args are 24 bytes");
static_assert(sizeof(nvshmemx_init_args_t) == 128, "init args are 128 bytes");
static_assert(sizeof(nvshmemx_init_attr_t) == 144, "init attr is 144 bytes");
static_assert(sizeof(nvshmem_team_config_t) == 64, "team config is 64 bytes");
#endif
#define NVSHMEMX_UNIQUEID_INITIALIZER { (1 << 16) + (int)sizeof(nvshmemx_uniqueid_t), {0} }
#define NVSHMEMX_UNIQUEID_ARGS_INITIALIZER { (1 << 16) + (int)sizeof(nvshmemx_uniqueid_args_t), NULL, -1, -1 }
#define NVSHMEMX_INIT_ARGS_INITIALIZER { (2 << 16) + (int)sizeof(nvshmemx_init_args_t), NVSHMEMX_UNIQUEID_ARGS_INITIALIZER, -1, {0} }
#define NVSHMEMX_INIT_ATTR_INITIALIZER { (2 << 16) + (int)sizeof(nvshmemx_init_attr_t), NULL, NVSHMEMX_INIT_ARGS_INITIALIZER }
#define NVSHMEM_TEAM_CONFIG_INITIALIZER { (2 << 16) + (int)sizeof(nvshmem_team_config_t), 0, 0, {0} }

/* ---------------------------------------------------------------- library set-up, exit and query */
void nvshmem_init(void);
int nvshmem_init_thread(int requested, int* provided);
int nvshmemx_init_attr(unsigned int flags, nvshmemx_init_attr_t* attr);
int nvshmemx_hostlib_init_attr(unsigned int flags, nvshmemx_init_attr_t* attr);
int nvshmemx_get_uniqueid(nvshmemx_uniqueid_t* id);
int nvshmemx_set_attr_uniqueid_args(int myrank, int nranks, const nvshmemx_uniqueid_t* id, nvshmemx_init_attr_t* attr);
int nvshmemx_init_status(void);
void nvshmem_finalize(void);
void nvshmemx_hostlib_finalize(void);
BSHMEM_HD void nvshmem_global_exit(int status);
void nvshmem_query_thread(int* provided);
BSHMEM_HD int nvshmem_my_pe(void);
BSHMEM_HD int nvshmem_n_pes(void);
void nvshmem_info_get_version(int* major, int* minor);
void nvshmem_info_get_name(char* name);
void nvshmemx_vendor_get_version_info(int* major, int* minor, int* patch);
int nvshmemx_cumodule_init(void* cumodule);   /* CUmodule */
int nvshmemx_cumodule_finalize(void* cumodule);
int nvshmemx_culibrary_init(void* culibrary); /* CUlibrary */
int nvshmemx_culibrary_finalize(void* culibrary);

/* ---------------------------------------------------------------- memory */
void* nvshmem_malloc(size_t size);
void* nvshmem_calloc(size_t count, size_t size);
void* nvshmem_align(size_t alignment, size_t size);
void nvshmem_free(void* ptr);
BSHMEM_HD void* nvshmem_ptr(const void* dest, int pe);
BSHMEM_HD void* nvshmemx_mc_ptr(nvshmem_team_t team, const void* ptr);
int nvshmemx_buffer_register(void* addr, size_t length);
int nvshmemx_buffer_unregister(void* addr);
void nvshmemx_buffer_unregister_all(void);
void* nvshmemx_buffer_register_symmetric(void* buf_ptr, size_t size, int flags);
int nvshmemx_buffer_unregister_symmetric(void* mmap_ptr, size_t size);

/* ---------------------------------------------------------------- teams */
BSHMEM_HD int nvshmem_team_my_pe(nvshmem_team_t team);
BSHMEM_HD int nvshmem_team_n_pes(nvshmem_team_t team);
void nvshmem_team_get_config(nvshmem_team_t team, nvshmem_team_config_t* config);
BSHMEM_HD int nvshmem_team_translate_pe(nvshmem_team_t src_team, int src_pe, nvshmem_team_t dest_team);
int nvshmem_team_split_strided(nvshmem_team_t parent, int pe_start, int pe_stride, int pe_size, const nvshmem_team_config_t* config, long config_mask, nvshmem_team_t* new_team);
int nvshmem_team_split_2d(nvshmem_team_t parent, int xrange, const nvshmem_team_config_t* xaxis_config, long xaxis_mask, nvshmem_team_t* xaxis_team,
                          const nvshmem_team_config_t* yaxis_config, long yaxis_mask, nvshmem_team_t* yaxis_team);
void nvshmem_team_destroy(nvshmem_team_t team);
int nvshmemx_team_get_uniqueid(nvshmemx_team_uniqueid_t* uniqueid);
int nvshmemx_team_init(nvshmem_team_t* team, nvshmem_team_config_t* config, long config_mask, int npes, int pe_idx_in_team);

/* ---------------------------------------------------------------- ordering, signals, waits */
BSHMEM_HD void nvshmem_quiet(void);
BSHMEM_HD void nvshmem_fence(void);
void nvshmemx_quiet_on_stream(cudaStream_t stream);
BSHMEM_HD uint64_t nvshmem_signal_fetch(uint64_t* sig_addr);
BSHMEM_HD void nvshmemx_signal_op(uint64_t* sig_addr, uint64_t signal, int sig_op, int pe);
void nvshmemx_signal_op_on_stream(uint64_t* sig_addr, uint64_t signal, int sig_op, int pe, cudaStream_t stream);
void nvshmemx_signal_wait_until_on_stream(uint64_t* sig_addr, int cmp, uint64_t cmp_value, cudaStream_t stream);

/* ---------------------------------------------------------------- untyped RMA */
BSHMEM_HD void nvshmem_putmem(void* dest, const void* source, size_t bytes, int pe);
BSHMEM_HD void nvshmem_getmem(void* dest, const void* source, size_t bytes, int pe);
BSHMEM_HD void nvshmem_putmem_nbi(void* dest, const void* source, size_t bytes, int pe);
BSHMEM_HD void nvshmem_getmem_nbi(void* dest, const void* source, size_t bytes, int pe);
void nvshmemx_putmem_on_stream(void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
void nvshmemx_getmem_on_stream(void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
void nvshmemx_putmem_nbi_on_stream(void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
void nvshmemx_getmem_nbi_on_stream(void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
void nvshmemx_putmem_signal_on_stream(void* dest, const void* source, size_t bytes, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe, cudaStream_t stream);
void nvshmemx_putmem_signal_nbi_on_stream(void* dest, const void* source, size_t bytes, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe, cudaStream_t stream);

/* ---------------------------------------------------------------- typed RMA: put/get/p/g/iput/iget, nbi, on_stream, signal */
#define BSHMEM_DECL_RMA(N, T)                                                                                          \
  BSHMEM_HD void nvshmem_##N##_p(T* dest, const T value, int pe);                                                                \
  BSHMEM_HD T nvshmem_##N##_g(const T* src, int pe);                                                                             \
  BSHMEM_HD void nvshmem_##N##_put(T* dest, const T* src, size_t nelems, int pe);                                                \
  BSHMEM_HD void nvshmem_##N##_get(T* dest, const T* src, size_t nelems, int pe);                                                \
  BSHMEM_HD void nvshmem_##N##_put_nbi(T* dest, const T* src, size_t nelems, int pe);                                            \
  BSHMEM_HD void nvshmem_##N##_get_nbi(T* dest, const T* src, size_t nelems, int pe);                                            \
  BSHMEM_HD void nvshmem_##N##_iput(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe);                 \
  BSHMEM_HD void nvshmem_##N##_iget(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe);                 \
  void nvshmemx_##N##_p_on_stream(T* dest, const T value, int pe, cudaStream_t s);                                     \
  T nvshmemx_##N##_g_on_stream(const T* src, int pe, cudaStream_t s);                                                  \
  void nvshmemx_##N##_put_on_stream(T* dest, const T* src, size_t nelems, int pe, cudaStream_t s);                     \
  void nvshmemx_##N##_get_on_stream(T* dest, const T* src, size_t nelems, int pe, cudaStream_t s);                     \
  void nvshmemx_##N##_put_nbi_on_stream(T* dest, const T* src, size_t nelems, int pe, cudaStream_t s);                 \
  void nvshmemx_##N##_get_nbi_on_stream(T* dest, const T* src, size_t nelems, int pe, cudaStream_t s);                 \
  void nvshmemx_##N##_iput_on_stream(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe, cudaStream_t s); \
  void nvshmemx_##N##_iget_on_stream(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe, cudaStream_t s); \
  void nvshmemx_##N##_put_signal_on_stream(T* dest, const T* src, size_t nelems, uint64_t* sig, uint64_t signal, int sig_op, int pe, cudaStream_t s); \
  void nvshmemx_##N##_put_signal_nbi_on_stream(T* dest, const T* src, size_t nelems, uint64_t* sig, uint64_t signal, int sig_op, int pe, cudaStream_t s);
BSHMEM_RMA_TYPES(BSHMEM_DECL_RMA)
#undef BSHMEM_DECL_RMA

#define BSHMEM_DECL_SIZED(BITS, T)                                                                                     \
  BSHMEM_HD void nvshmem_put##BITS(void* dest, const void* src, size_t nelems, int pe);                                          \
  BSHMEM_HD void nvshmem_get##BITS(void* dest, const void* src, size_t nelems, int pe);                                          \
  BSHMEM_HD void nvshmem_put##BITS##_nbi(void* dest, const void* src, size_t nelems, int pe);                                    \
  BSHMEM_HD void nvshmem_get##BITS##_nbi(void* dest, const void* src, size_t nelems, int pe);                                    \
  BSHMEM_HD void nvshmem_iput##BITS(void* dest, const void* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe);           \
  BSHMEM_HD void nvshmem_iget##BITS(void* dest, const void* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe);           \
  void nvshmemx_put##BITS##_on_stream(void* dest, const void* src, size_t nelems, int pe, cudaStream_t s);             \
  void nvshmemx_get##BITS##_on_stream(void* dest, const void* src, size_t nelems, int pe, cudaStream_t s);             \
  void nvshmemx_put##BITS##_signal_on_stream(void* dest, const void* src, size_t nelems, uint64_t* sig, uint64_t signal, int sig_op, int pe, cudaStream_t s); \
  void nvshmemx_put##BITS##_signal_nbi_on_stream(void* dest, const void* src, size_t nelems, uint64_t* sig, uint64_t signal, int sig_op, int pe, cudaStream_t s); \
  void nvshmemx_put##BITS##_nbi_on_stream(void* dest, const void* src, size_t nelems, int pe, cudaStream_t s);         \
  void nvshmemx_get##BITS##_nbi_on_stream(void* dest, const void* src, size_t nelems, int pe, cudaStream_t s);         \
  void nvshmemx_iput##BITS##_on_stream(void* dest, const void* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe, cudaStream_t s); \
  void nvshmemx_iget##BITS##_on_stream(void* dest, const void* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe, cudaStream_t s);
BSHMEM_SIZES(BSHMEM_DECL_SIZED)
#undef BSHMEM_DECL_SIZED

/* ---------------------------------------------------------------- on-stream waits */
#define BSHMEM_DECL_WAIT(N, T)                                                                                         \
  void nvshmemx_##N##_wait_until_on_stream(T* ivar, int cmp, T cmp_value, cudaStream_t s);                             \
  void nvshmemx_##N##_wait_until_all_on_stream(T* ivars, size_t nelems, const int* status, int cmp, T cmp_value, cudaStream_t s); \
  void nvshmemx_##N##_wait_until_all_vector_on_stream(T* ivars, size_t nelems, const int* status, int cmp, T* cmp_values, cudaStream_t s);
BSHMEM_WAIT_TYPES(BSHMEM_DECL_WAIT)
#undef BSHMEM_DECL_WAIT

/* ---------------------------------------------------------------- host atomics (carried out by a one-thread kernel) */
#define BSHMEM_DECL_AMO_STD(N, T)                                      \
  BSHMEM_HD void nvshmem_##N##_atomic_inc(T* target, int pe);                    \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch_inc(T* target, int pe);                 \
  BSHMEM_HD void nvshmem_##N##_atomic_add(T* target, T value, int pe);           \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch_add(T* target, T value, int pe);        \
  BSHMEM_HD T nvshmem_##N##_atomic_compare_swap(T* target, T cond, T value, int pe);
#define BSHMEM_DECL_AMO_EXT(N, T)                                      \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch(const T* target, int pe);               \
  BSHMEM_HD void nvshmem_##N##_atomic_set(T* target, T value, int pe);           \
  BSHMEM_HD T nvshmem_##N##_atomic_swap(T* target, T value, int pe);
#define BSHMEM_DECL_AMO_BIT(N, T)                                      \
  BSHMEM_HD void nvshmem_##N##_atomic_and(T* target, T value, int pe);           \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch_and(T* target, T value, int pe);        \
  BSHMEM_HD void nvshmem_##N##_atomic_or(T* target, T value, int pe);            \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch_or(T* target, T value, int pe);         \
  BSHMEM_HD void nvshmem_##N##_atomic_xor(T* target, T value, int pe);           \
  BSHMEM_HD T nvshmem_##N##_atomic_fetch_xor(T* target, T value, int pe);
BSHMEM_STANDARD_AMO_TYPES(BSHMEM_DECL_AMO_STD)
BSHMEM_EXTENDED_AMO_TYPES(BSHMEM_DECL_AMO_EXT)
BSHMEM_BITWISE_AMO_TYPES(BSHMEM_DECL_AMO_BIT)
#undef BSHMEM_DECL_AMO_STD
#undef BSHMEM_DECL_AMO_EXT
#undef BSHMEM_DECL_AMO_BIT

/* ---------------------------------------------------------------- collectives: blocking and on-stream */
BSHMEM_HD void nvshmem_barrier_all(void);
BSHMEM_HD int nvshmem_barrier(nvshmem_team_t team);
BSHMEM_HD void nvshmem_sync_all(void);
BSHMEM_HD int nvshmem_team_sync(nvshmem_team_t team);
void nvshmemx_barrier_all_on_stream(cudaStream_t stream);
int nvshmemx_barrier_on_stream(nvshmem_team_t team, cudaStream_t stream);
void nvshmemx_sync_all_on_stream(cudaStream_t stream);
int nvshmemx_team_sync_on_stream(nvshmem_team_t team, cudaStream_t stream);
BSHMEM_HD int nvshmem_alltoallmem(nvshmem_team_t team, void* dest, const void* src, size_t bytes);
BSHMEM_HD int nvshmem_fcollectmem(nvshmem_team_t team, void* dest, const void* src, size_t bytes);
BSHMEM_HD int nvshmem_broadcastmem(nvshmem_team_t team, void* dest, const void* src, size_t bytes, int root);
int nvshmemx_alltoallmem_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t bytes, cudaStream_t s);
int nvshmemx_fcollectmem_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t bytes, cudaStream_t s);
int nvshmemx_broadcastmem_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t bytes, int root, cudaStream_t s);
int nvshmemx_double2_maxloc_reduce_on_stream(nvshmem_team_t team, double2* dest, const double2* src, size_t nreduce, cudaStream_t s);

#define BSHMEM_DECL_COLL(N, T)                                                                                         \
  BSHMEM_HD int nvshmem_##N##_alltoall(nvshmem_team_t team, T* dest, const T* src, size_t nelems);                               \
  BSHMEM_HD int nvshmem_##N##_fcollect(nvshmem_team_t team, T* dest, const T* src, size_t nelems);                               \
  BSHMEM_HD int nvshmem_##N##_broadcast(nvshmem_team_t team, T* dest, const T* src, size_t nelems, int root);                    \
  int nvshmemx_##N##_alltoall_on_stream(nvshmem_team_t team, T* dest, const T* src, size_t nelems, cudaStream_t s);    \
  int nvshmemx_##N##_fcollect_on_stream(nvshmem_team_t team, T* dest, const T* src, size_t nelems, cudaStream_t s);    \
  int nvshmemx_##N##_broadcast_on_stream(nvshmem_team_t team, T* dest, const T* src, size_t nelems, int root, cudaStream_t s);
BSHMEM_RMA_TYPES(BSHMEM_DECL_COLL)
#undef BSHMEM_DECL_COLL

#define BSHMEM_DECL_REDUCE_OP(N, T, OPNAME)                                                                            \
  BSHMEM_HD int nvshmem_##N##_##OPNAME##_reduce(nvshmem_team_t team, T* dest, const T* src, size_t nreduce);                     \
  BSHMEM_HD int nvshmem_##N##_##OPNAME##_reducescatter(nvshmem_team_t team, T* dest, const T* src, size_t nreduce);              \
  int nvshmemx_##N##_##OPNAME##_reduce_on_stream(nvshmem_team_t team, T* dest, const T* src, size_t nreduce, cudaStream_t s); \
  int nvshmemx_##N##_##OPNAME##_reducescatter_on_stream(nvshmem_team_t team, T* dest, const T* src, size_t nreduce, cudaStream_t s);
#define BSHMEM_DECL_BITWISE(N, T) BSHMEM_DECL_REDUCE_OP(N, T, and) BSHMEM_DECL_REDUCE_OP(N, T, or) BSHMEM_DECL_REDUCE_OP(N, T, xor)
#define BSHMEM_DECL_ARITH(N, T) BSHMEM_DECL_REDUCE_OP(N, T, min) BSHMEM_DECL_REDUCE_OP(N, T, max) BSHMEM_DECL_REDUCE_OP(N, T, sum) BSHMEM_DECL_REDUCE_OP(N, T, prod)
BSHMEM_BITWISE_REDUCE_TYPES(BSHMEM_DECL_BITWISE)
BSHMEM_STANDARD_REDUCE_TYPES(BSHMEM_DECL_ARITH)
#undef BSHMEM_DECL_BITWISE
#undef BSHMEM_DECL_ARITH
#undef BSHMEM_DECL_REDUCE_OP

/* ---------------------------------------------------------------- queue pairs
 * Handles for the nvshmemx_qp_* device calls.  Peers reached by loads and stores have no queues: every handle
 * names the same (only) path, and an MPI communicator cannot be used to initialise (no MPI bootstrap is built). */
typedef int nvshmemx_qp_handle_t;
enum { NVSHMEMX_QP_HOST = 0, NVSHMEMX_QP_DEFAULT = 1, NVSHMEMX_QP_ANY = 0x7fffffff, NVSHMEMX_QP_ALL = 0x7fffffff };
int nvshmemx_qp_create(int num_qps, nvshmemx_qp_handle_t** out_qp_array);
int nvshmemx_set_attr_mpi_comm_args(void* mpi_comm, nvshmemx_init_attr_t* attr);

/* ---------------------------------------------------------------- collective launch */
int nvshmemx_collective_launch(const void* func, dim3 grid_dims, dim3 block_dims, void** args, size_t shared_mem, cudaStream_t stream);
int nvshmemx_collective_launch_query_gridsize(const void* func, dim3 block_dims, void** args, size_t shared_mem, int* gridsize);

/* ---------------------------------------------------------------- extensions of this library (no NVSHMEM counterpart) */
/* Fills the device-state copy of every library with device code loaded so far.  Initialisation and
 * every later API call do this on their own; call it after loading such a library at run time when
 * its kernels are launched before any other call into this library. */
void nvshmemx_b200_module_sync(void);
/* On-stream alltoall / fcollect / broadcast of at least `min_bytes` (whole buffer) use the copy engines from now on
 * (0 = never, the default; also NVSHMEM_CE_COLLECTIVES_MIN_BYTES).  Call it with the same value on every PE. */
void nvshmemx_b200_set_ce_collectives(size_t min_bytes);

#if defined(__cplusplus) && !defined(BSHMEM_NO_INLINE_LAUNCH)
/* A kernel's host-side handle belongs to the CUDA runtime instance of the program that defines it.  A program
 * that links the CUDA runtime statically (nvcc's default) has its own instance, so the occupancy query and the
 * cooperative launch are compiled into the caller; the library is only asked to refresh the device state. */
static inline int bshmemx_inline_collective_launch_query_gridsize(const void* func, dim3 block, void** args, size_t smem, int* gridsize) {
  (void)args;
  if (!gridsize) return NVSHMEMX_ERROR_INVALID_VALUE;
  int per_sm = 0, dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return NVSHMEMX_ERROR_INTERNAL;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, func, (int)(block.x * block.y * block.z), smem) != cudaSuccess) return NVSHMEMX_ERROR_INTERNAL;
  *gridsize = per_sm * sms;
  return NVSHMEMX_SUCCESS;
}
static inline int bshmemx_inline_collective_launch(const void* func, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t stream) {
  if (nvshmemx_init_status() < NVSHMEM_STATUS_IS_INITIALIZED) return NVSHMEMX_ERROR_INVALID_VALUE;
  nvshmemx_b200_module_sync();
  int max_grid = 0;
  if (bshmemx_inline_collective_launch_query_gridsize(func, block, args, smem, &max_grid) != NVSHMEMX_SUCCESS) return NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;
  if (grid.x == 0) grid = dim3((unsigned)max_grid, 1, 1);
  if ((int)(grid.x * grid.y * grid.z) > max_grid) return NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;  /* the CTAs could not all be resident */
  return cudaLaunchCooperativeKernel(func, grid, block, args, smem, stream) == cudaSuccess ? NVSHMEMX_SUCCESS : NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;
}
#define nvshmemx_collective_launch bshmemx_inline_collective_launch
#define nvshmemx_collective_launch_query_gridsize bshmemx_inline_collective_launch_query_gridsize
#endif
/* Error bits recorded by device code since the last clear (BSHMEM_ERR_*): bounded waits
 * report a time-out here instead of hanging the GPU. */
uint32_t nvshmemx_b200_error_bits(void);
void nvshmemx_b200_clear_errors(void);
/* Copies the last time-out record into the caller's struct; returns the count so far. */
uint32_t nvshmemx_b200_timeout_info(bshmemi_status_t* out);
/* Overrides NVSHMEM_WAIT_TIMEOUT_MS at run time (tests use a short bound). */
void nvshmemx_b200_set_wait_timeout_ms(long ms);
/* One-line description of the probed topology, valid until the next call. */
const char* nvshmemx_b200_topology(void);
/* Heap facts: 0 base of the local window, 1 stride, 2 backed bytes, 3 multicast base, 4 chunks, 5 bytes in use,
 * 6 digest of the allocation history, 7 whether the heap is GPU memory. */
uint64_t nvshmemx_b200_heap_info(int what);
/* Detaches this PE from every NVLink multicast object (unmap, unbind, release) without any collective step.
 * For a process that is about to leave abnormally: peers' GPUs must not be left with a member that vanished
 * while bound.  NVLS collectives are off on this PE afterwards. */
void nvshmemx_b200_release_multicast(void);
/* Explicit algorithm choice for benchmarks (0 = automatic). */
int nvshmemx_b200_reduce_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t n, int dtype, int op, int algo, cudaStream_t s);
int nvshmemx_b200_reducescatter_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t n, int dtype, int op, int algo, cudaStream_t s);
int nvshmemx_b200_fcollect_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t bytes, int algo, cudaStream_t s);
int nvshmemx_b200_broadcast_on_stream(nvshmem_team_t team, void* dest, const void* src, size_t bytes, int root, int algo, cudaStream_t s);
/* Initialisation from explicit arguments, the form the Python layer uses. */
int nvshmemx_b200_init_uid(const nvshmemx_uniqueid_t* id, int rank, int nranks, int device);

#ifdef __cplusplus
}
#endif
