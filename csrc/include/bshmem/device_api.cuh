// Device-side public API: the nvshmem_* / nvshmemx_* names callable from CUDA
// kernels, generated from the type tables and mapped onto the templates of
// device.cuh and coll.cuh.  Scope naming follows NVSHMEM: no suffix = calling
// thread, nvshmemx_*_warp, nvshmemx_*_block (and _warpgroup for barriers and
// tile collectives).  Definitions are only visible to the device compilation
// pass; the host pass sees the declarations of nvshmem_host.h and links against
// the host library
// (reference: src/include/device/nvshmem_defines.h, nvshmemx_defines.h,
//  nvshmem_coll_defines.cuh, nvshmemx_coll_defines.cuh).
#pragma once
#include "../nvshmem_host.h"
#include "coll.cuh"
#include "device.cuh"

// Functions that also exist on the host are defined for the device pass only (the host pass
// binds the name to the host library); device-only functions are defined in both passes so
// that kernels parse in the host pass too.
#ifdef __CUDA_ARCH__
#define BSHMEM_DEV(ret, name, params, ...) extern "C" __host__ __device__ __forceinline__ ret name params __VA_ARGS__
#else
#define BSHMEM_DEV(ret, name, params, ...)
#endif
#define BSHMEM_DEVX extern "C" __device__ __forceinline__

// ------------------------------------------------------------------ queries, ordering
BSHMEM_DEV(int, nvshmem_my_pe, (void), { return bshmem::my_pe(); })
BSHMEM_DEV(int, nvshmem_n_pes, (void), { return bshmem::n_pes(); })
BSHMEM_DEV(void*, nvshmem_ptr, (const void* dest, int pe), { return bshmem::ptr(dest, pe); })
BSHMEM_DEV(void*, nvshmemx_mc_ptr, (nvshmem_team_t team, const void* p), {
  const bshmemi_team_t* t = bshmem::team_ptr(team);
  return t && t->has_nvls && bshmem::in_heap(p) ? (void*)(t->mc_base + ((uint64_t)p - bshmemi_state_d.heap_base)) : nullptr;
})
BSHMEM_DEV(int, nvshmem_team_my_pe, (nvshmem_team_t team), { return bshmem::team_my_pe(team); })
BSHMEM_DEV(int, nvshmem_team_n_pes, (nvshmem_team_t team), { return bshmem::team_n_pes(team); })
BSHMEM_DEV(int, nvshmem_team_translate_pe, (nvshmem_team_t s, int pe, nvshmem_team_t d), { return bshmem::team_translate_pe(s, pe, d); })
BSHMEM_DEV(void, nvshmem_quiet, (void), { bshmem::fence_sys(); })
BSHMEM_DEV(void, nvshmem_fence, (void), { bshmem::fence_sys(); })
BSHMEM_DEV(void, nvshmem_global_exit, (int status), { bshmem::global_exit(status); })
BSHMEM_DEVX void nvshmemx_quiet_warp(void) { bshmem::quiet<bshmem::SCOPE_WARP>(); }
BSHMEM_DEVX void nvshmemx_quiet_block(void) { bshmem::quiet<bshmem::SCOPE_BLOCK>(); }
BSHMEM_DEVX void nvshmemx_fence_warp(void) { bshmem::quiet<bshmem::SCOPE_WARP>(); }
BSHMEM_DEVX void nvshmemx_fence_block(void) { bshmem::quiet<bshmem::SCOPE_BLOCK>(); }
// Error bits recorded so far by device code on this PE (bounded waits report here).
BSHMEM_DEVX unsigned nvshmemx_b200_device_error_bits(void) { return bshmem::error_bits(); }

// ------------------------------------------------------------------ signals
BSHMEM_DEV(uint64_t, nvshmem_signal_fetch, (uint64_t* sig_addr), { return bshmem::signal_fetch(sig_addr); })
BSHMEM_DEV(void, nvshmemx_signal_op, (uint64_t* sig_addr, uint64_t signal, int sig_op, int pe), { bshmem::signal_op(sig_addr, signal, sig_op, pe); })
BSHMEM_DEVX uint64_t nvshmem_signal_wait_until(uint64_t* sig_addr, int cmp, uint64_t cmp_val) {
  bshmem::wait_until<uint64_t>(sig_addr, cmp, cmp_val, BSHMEM_WHERE_SIGNAL_WAIT);
  return *(volatile uint64_t*)sig_addr;
}

// ------------------------------------------------------------------ untyped RMA, all scopes
BSHMEM_DEV(void, nvshmem_putmem, (void* d, const void* s, size_t n, int pe), { bshmem::putmem<bshmem::SCOPE_THREAD>(d, s, n, pe); })
BSHMEM_DEV(void, nvshmem_getmem, (void* d, const void* s, size_t n, int pe), { bshmem::getmem<bshmem::SCOPE_THREAD>(d, s, n, pe); })
BSHMEM_DEV(void, nvshmem_putmem_nbi, (void* d, const void* s, size_t n, int pe), { bshmem::putmem_nbi<bshmem::SCOPE_THREAD>(d, s, n, pe); })
BSHMEM_DEV(void, nvshmem_getmem_nbi, (void* d, const void* s, size_t n, int pe), { bshmem::getmem_nbi<bshmem::SCOPE_THREAD>(d, s, n, pe); })
BSHMEM_DEVX void nvshmem_putmem_signal(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n, sig, v, op, pe); }
BSHMEM_DEVX void nvshmem_putmem_signal_nbi(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n, sig, v, op, pe); }
#define BSHMEM_DEV_MEM_SCOPED(SUF, SC)                                                                                                   \
  BSHMEM_DEVX void nvshmemx_putmem_##SUF(void* d, const void* s, size_t n, int pe) { bshmem::putmem<SC>(d, s, n, pe); }                  \
  BSHMEM_DEVX void nvshmemx_getmem_##SUF(void* d, const void* s, size_t n, int pe) { bshmem::getmem<SC>(d, s, n, pe); }                  \
  BSHMEM_DEVX void nvshmemx_putmem_nbi_##SUF(void* d, const void* s, size_t n, int pe) { bshmem::putmem_nbi<SC>(d, s, n, pe); }          \
  BSHMEM_DEVX void nvshmemx_getmem_nbi_##SUF(void* d, const void* s, size_t n, int pe) { bshmem::getmem_nbi<SC>(d, s, n, pe); }          \
  BSHMEM_DEVX void nvshmemx_putmem_signal_##SUF(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<SC>(d, s, n, sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_putmem_signal_nbi_##SUF(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<SC>(d, s, n, sig, v, op, pe); }
BSHMEM_DEV_MEM_SCOPED(warp, bshmem::SCOPE_WARP)
BSHMEM_DEV_MEM_SCOPED(block, bshmem::SCOPE_BLOCK)
#undef BSHMEM_DEV_MEM_SCOPED

// ------------------------------------------------------------------ typed RMA
#define BSHMEM_DEV_RMA(N, T)                                                                                                             \
  BSHMEM_DEV(void, nvshmem_##N##_p, (T* dest, const T value, int pe), { bshmem::p<T>(dest, value, pe); })                                     \
  BSHMEM_DEV(T, nvshmem_##N##_g, (const T* src, int pe), { return bshmem::g<T>(src, pe); })                                                   \
  BSHMEM_DEV(void, nvshmem_##N##_put, (T* d, const T* s, size_t n, int pe), { bshmem::putmem<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); }) \
  BSHMEM_DEV(void, nvshmem_##N##_get, (T* d, const T* s, size_t n, int pe), { bshmem::getmem<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); }) \
  BSHMEM_DEV(void, nvshmem_##N##_put_nbi, (T* d, const T* s, size_t n, int pe), { bshmem::putmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); }) \
  BSHMEM_DEV(void, nvshmem_##N##_get_nbi, (T* d, const T* s, size_t n, int pe), { bshmem::getmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); }) \
  BSHMEM_DEV(void, nvshmem_##N##_iput, (T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe), { bshmem::iput<T, bshmem::SCOPE_THREAD>(d, s, dst, sst, n, pe); }) \
  BSHMEM_DEV(void, nvshmem_##N##_iget, (T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe), { bshmem::iget<T, bshmem::SCOPE_THREAD>(d, s, dst, sst, n, pe); }) \
  BSHMEM_DEVX void nvshmem_##N##_put_signal(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmem_##N##_put_signal_nbi(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), sig, v, op, pe); }
BSHMEM_RMA_TYPES(BSHMEM_DEV_RMA)
#undef BSHMEM_DEV_RMA

#define BSHMEM_DEV_RMA_SCOPED(N, T, SUF, SC)                                                                                             \
  BSHMEM_DEVX void nvshmemx_##N##_put_##SUF(T* d, const T* s, size_t n, int pe) { bshmem::putmem<SC>(d, s, n * sizeof(T), pe); }         \
  BSHMEM_DEVX void nvshmemx_##N##_get_##SUF(T* d, const T* s, size_t n, int pe) { bshmem::getmem<SC>(d, s, n * sizeof(T), pe); }         \
  BSHMEM_DEVX void nvshmemx_##N##_put_nbi_##SUF(T* d, const T* s, size_t n, int pe) { bshmem::putmem_nbi<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_##N##_get_nbi_##SUF(T* d, const T* s, size_t n, int pe) { bshmem::getmem_nbi<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_##N##_iput_##SUF(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iput<T, SC>(d, s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmemx_##N##_iget_##SUF(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iget<T, SC>(d, s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmemx_##N##_put_signal_##SUF(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<SC>(d, s, n * sizeof(T), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_##N##_put_signal_nbi_##SUF(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<SC>(d, s, n * sizeof(T), sig, v, op, pe); }
#define BSHMEM_DEV_RMA_WARP(N, T) BSHMEM_DEV_RMA_SCOPED(N, T, warp, bshmem::SCOPE_WARP)
#define BSHMEM_DEV_RMA_BLOCK(N, T) BSHMEM_DEV_RMA_SCOPED(N, T, block, bshmem::SCOPE_BLOCK)
BSHMEM_RMA_TYPES(BSHMEM_DEV_RMA_WARP)
BSHMEM_RMA_TYPES(BSHMEM_DEV_RMA_BLOCK)
#undef BSHMEM_DEV_RMA_WARP
#undef BSHMEM_DEV_RMA_BLOCK
#undef BSHMEM_DEV_RMA_SCOPED

#define BSHMEM_DEV_SIZED(BITS, T)                                                                                                        \
  BSHMEM_DEV(void, nvshmem_put##BITS, (void* d, const void* s, size_t n, int pe), { bshmem::putmem<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), pe); }) \
  BSHMEM_DEV(void, nvshmem_get##BITS, (void* d, const void* s, size_t n, int pe), { bshmem::getmem<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), pe); }) \
  BSHMEM_DEV(void, nvshmem_put##BITS##_nbi, (void* d, const void* s, size_t n, int pe), { bshmem::putmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), pe); }) \
  BSHMEM_DEV(void, nvshmem_get##BITS##_nbi, (void* d, const void* s, size_t n, int pe), { bshmem::getmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), pe); }) \
  BSHMEM_DEV(void, nvshmem_iput##BITS, (void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe), { bshmem::iput<T, bshmem::SCOPE_THREAD>((T*)d, (const T*)s, dst, sst, n, pe); }) \
  BSHMEM_DEV(void, nvshmem_iget##BITS, (void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe), { bshmem::iget<T, bshmem::SCOPE_THREAD>((T*)d, (const T*)s, dst, sst, n, pe); }) \
  BSHMEM_DEVX void nvshmemx_put##BITS##_warp(void* d, const void* s, size_t n, int pe) { bshmem::putmem<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_block(void* d, const void* s, size_t n, int pe) { bshmem::putmem<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_get##BITS##_warp(void* d, const void* s, size_t n, int pe) { bshmem::getmem<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_get##BITS##_block(void* d, const void* s, size_t n, int pe) { bshmem::getmem<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_nbi_warp(void* d, const void* s, size_t n, int pe) { bshmem::putmem_nbi<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_nbi_block(void* d, const void* s, size_t n, int pe) { bshmem::putmem_nbi<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_get##BITS##_nbi_warp(void* d, const void* s, size_t n, int pe) { bshmem::getmem_nbi<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmemx_get##BITS##_nbi_block(void* d, const void* s, size_t n, int pe) { bshmem::getmem_nbi<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), pe); } \
  BSHMEM_DEVX void nvshmem_put##BITS##_signal(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_signal_warp(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_signal_block(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), sig, v, op, pe); }
BSHMEM_SIZES(BSHMEM_DEV_SIZED)
#undef BSHMEM_DEV_SIZED

// ------------------------------------------------------------------ wait / test families
#define BSHMEM_DEV_WAIT(N, T)                                                                                                            \
  BSHMEM_DEVX void nvshmem_##N##_wait_until(T* ivar, int cmp, T v) { bshmem::wait_until<T>(ivar, cmp, v); }                              \
  BSHMEM_DEVX void nvshmem_##N##_wait_until_all(T* ivars, size_t n, const int* status, int cmp, T v) { bshmem::wait_until_all<T>(ivars, n, status, cmp, nullptr, v); } \
  BSHMEM_DEVX size_t nvshmem_##N##_wait_until_any(T* ivars, size_t n, const int* status, int cmp, T v) { return bshmem::wait_until_any<T>(ivars, n, status, cmp, nullptr, v); } \
  BSHMEM_DEVX size_t nvshmem_##N##_wait_until_some(T* ivars, size_t n, size_t* idx, const int* status, int cmp, T v) { return bshmem::wait_until_some<T>(ivars, n, idx, status, cmp, nullptr, v); } \
  BSHMEM_DEVX void nvshmem_##N##_wait_until_all_vector(T* ivars, size_t n, const int* status, int cmp, T* vs) { bshmem::wait_until_all<T>(ivars, n, status, cmp, vs, (T)0); } \
  BSHMEM_DEVX size_t nvshmem_##N##_wait_until_any_vector(T* ivars, size_t n, const int* status, int cmp, T* vs) { return bshmem::wait_until_any<T>(ivars, n, status, cmp, vs, (T)0); } \
  BSHMEM_DEVX size_t nvshmem_##N##_wait_until_some_vector(T* ivars, size_t n, size_t* idx, const int* status, int cmp, T* vs) { return bshmem::wait_until_some<T>(ivars, n, idx, status, cmp, vs, (T)0); } \
  BSHMEM_DEVX int nvshmem_##N##_test(T* ivar, int cmp, T v) { return bshmem::test<T>(ivar, cmp, v); }                                    \
  BSHMEM_DEVX int nvshmem_##N##_test_all(T* ivars, size_t n, const int* status, int cmp, T v) { return bshmem::test_all<T>(ivars, n, status, cmp, nullptr, v); } \
  BSHMEM_DEVX size_t nvshmem_##N##_test_any(T* ivars, size_t n, const int* status, int cmp, T v) { return bshmem::test_any<T>(ivars, n, status, cmp, nullptr, v); } \
  BSHMEM_DEVX size_t nvshmem_##N##_test_some(T* ivars, size_t n, size_t* idx, const int* status, int cmp, T v) { return bshmem::test_some<T>(ivars, n, idx, status, cmp, nullptr, v); } \
  BSHMEM_DEVX int nvshmem_##N##_test_all_vector(T* ivars, size_t n, const int* status, int cmp, T* vs) { return bshmem::test_all<T>(ivars, n, status, cmp, vs, (T)0); } \
  BSHMEM_DEVX size_t nvshmem_##N##_test_any_vector(T* ivars, size_t n, const int* status, int cmp, T* vs) { return bshmem::test_any<T>(ivars, n, status, cmp, vs, (T)0); } \
  BSHMEM_DEVX size_t nvshmem_##N##_test_some_vector(T* ivars, size_t n, size_t* idx, const int* status, int cmp, T* vs) { return bshmem::test_some<T>(ivars, n, idx, status, cmp, vs, (T)0); }
BSHMEM_WAIT_TYPES(BSHMEM_DEV_WAIT)
#undef BSHMEM_DEV_WAIT

// ------------------------------------------------------------------ atomics
#define BSHMEM_DEV_AMO_STD(N, T)                                                                                                         \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_inc, (T* t, int pe), { bshmem::atomic_add<T>(t, (T)1, pe); })                                         \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch_inc, (T* t, int pe), { return bshmem::atomic_fetch_add<T>(t, (T)1, pe); })                         \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_add, (T* t, T v, int pe), { bshmem::atomic_add<T>(t, v, pe); })                                       \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch_add, (T* t, T v, int pe), { return bshmem::atomic_fetch_add<T>(t, v, pe); })                       \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_compare_swap, (T* t, T c, T v, int pe), { return bshmem::atomic_compare_swap<T>(t, c, v, pe); })
#define BSHMEM_DEV_AMO_EXT(N, T)                                                                                                         \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch, (const T* t, int pe), { return bshmem::atomic_fetch<T>(t, pe); })                                 \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_set, (T* t, T v, int pe), { bshmem::atomic_set<T>(t, v, pe); })                                       \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_swap, (T* t, T v, int pe), { return bshmem::atomic_swap<T>(t, v, pe); })
#define BSHMEM_DEV_AMO_BIT(N, T)                                                                                                         \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_and, (T* t, T v, int pe), { (void)bshmem::atomic_fetch_and<T>(t, v, pe); })                           \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch_and, (T* t, T v, int pe), { return bshmem::atomic_fetch_and<T>(t, v, pe); })                       \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_or, (T* t, T v, int pe), { (void)bshmem::atomic_fetch_or<T>(t, v, pe); })                             \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch_or, (T* t, T v, int pe), { return bshmem::atomic_fetch_or<T>(t, v, pe); })                         \
  BSHMEM_DEV(void, nvshmem_##N##_atomic_xor, (T* t, T v, int pe), { (void)bshmem::atomic_fetch_xor<T>(t, v, pe); })                           \
  BSHMEM_DEV(T, nvshmem_##N##_atomic_fetch_xor, (T* t, T v, int pe), { return bshmem::atomic_fetch_xor<T>(t, v, pe); })
BSHMEM_STANDARD_AMO_TYPES(BSHMEM_DEV_AMO_STD)
BSHMEM_EXTENDED_AMO_TYPES(BSHMEM_DEV_AMO_EXT)
BSHMEM_BITWISE_AMO_TYPES(BSHMEM_DEV_AMO_BIT)
#undef BSHMEM_DEV_AMO_STD
#undef BSHMEM_DEV_AMO_EXT
#undef BSHMEM_DEV_AMO_BIT

// ------------------------------------------------------------------ barriers
BSHMEM_DEV(void, nvshmem_barrier_all, (void), { bshmem::team_barrier<bshmem::SCOPE_THREAD>(bshmem::team_ptr(0)); })
BSHMEM_DEV(int, nvshmem_barrier, (nvshmem_team_t team), { return bshmem::team_barrier<bshmem::SCOPE_THREAD>(bshmem::team_ptr(team)); })
BSHMEM_DEV(void, nvshmem_sync_all, (void), { bshmem::team_sync<bshmem::SCOPE_THREAD>(bshmem::team_ptr(0)); })
BSHMEM_DEV(int, nvshmem_team_sync, (nvshmem_team_t team), { return bshmem::team_sync<bshmem::SCOPE_THREAD>(bshmem::team_ptr(team)); })
#define BSHMEM_DEV_BARRIER_SCOPED(SUF, SC)                                                                                               \
  BSHMEM_DEVX void nvshmemx_barrier_all_##SUF(void) { bshmem::team_barrier<SC>(bshmem::team_ptr(0)); }                                   \
  BSHMEM_DEVX int nvshmemx_barrier_##SUF(nvshmem_team_t team) { return bshmem::team_barrier<SC>(bshmem::team_ptr(team)); }               \
  BSHMEM_DEVX void nvshmemx_sync_all_##SUF(void) { bshmem::team_sync<SC>(bshmem::team_ptr(0)); }                                         \
  BSHMEM_DEVX int nvshmemx_team_sync_##SUF(nvshmem_team_t team) { return bshmem::team_sync<SC>(bshmem::team_ptr(team)); }
BSHMEM_DEV_BARRIER_SCOPED(warp, bshmem::SCOPE_WARP)
BSHMEM_DEV_BARRIER_SCOPED(warpgroup, bshmem::SCOPE_WARPGROUP)
BSHMEM_DEV_BARRIER_SCOPED(block, bshmem::SCOPE_BLOCK)
#undef BSHMEM_DEV_BARRIER_SCOPED

// ------------------------------------------------------------------ collectives
BSHMEM_DEV(int, nvshmem_alltoallmem, (nvshmem_team_t team, void* d, const void* s, size_t bytes), { return bshmem::alltoall<char, bshmem::SCOPE_THREAD>(team, (char*)d, (const char*)s, bytes); })
BSHMEM_DEV(int, nvshmem_fcollectmem, (nvshmem_team_t team, void* d, const void* s, size_t bytes), { return bshmem::fcollect<char, bshmem::SCOPE_THREAD>(team, (char*)d, (const char*)s, bytes); })
BSHMEM_DEV(int, nvshmem_broadcastmem, (nvshmem_team_t team, void* d, const void* s, size_t bytes, int root), { return bshmem::broadcast<char, bshmem::SCOPE_THREAD>(team, (char*)d, (const char*)s, bytes, root); })
#define BSHMEM_DEV_COLL(N, T)                                                                                                            \
  BSHMEM_DEV(int, nvshmem_##N##_alltoall, (nvshmem_team_t team, T* d, const T* s, size_t n), { return bshmem::alltoall<T, bshmem::SCOPE_THREAD>(team, d, s, n); }) \
  BSHMEM_DEV(int, nvshmem_##N##_fcollect, (nvshmem_team_t team, T* d, const T* s, size_t n), { return bshmem::fcollect<T, bshmem::SCOPE_THREAD>(team, d, s, n); }) \
  BSHMEM_DEV(int, nvshmem_##N##_broadcast, (nvshmem_team_t team, T* d, const T* s, size_t n, int root), { return bshmem::broadcast<T, bshmem::SCOPE_THREAD>(team, d, s, n, root); })
BSHMEM_RMA_TYPES(BSHMEM_DEV_COLL)
#undef BSHMEM_DEV_COLL
#define BSHMEM_DEV_COLL_SCOPED(N, T, SUF, SC)                                                                                            \
  BSHMEM_DEVX int nvshmemx_##N##_alltoall_##SUF(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::alltoall<T, SC>(team, d, s, n); } \
  BSHMEM_DEVX int nvshmemx_##N##_fcollect_##SUF(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::fcollect<T, SC>(team, d, s, n); } \
  BSHMEM_DEVX int nvshmemx_##N##_broadcast_##SUF(nvshmem_team_t team, T* d, const T* s, size_t n, int root) { return bshmem::broadcast<T, SC>(team, d, s, n, root); }
#define BSHMEM_DEV_COLL_WARP(N, T) BSHMEM_DEV_COLL_SCOPED(N, T, warp, bshmem::SCOPE_WARP)
#define BSHMEM_DEV_COLL_BLOCK(N, T) BSHMEM_DEV_COLL_SCOPED(N, T, block, bshmem::SCOPE_BLOCK)
BSHMEM_RMA_TYPES(BSHMEM_DEV_COLL_WARP)
BSHMEM_RMA_TYPES(BSHMEM_DEV_COLL_BLOCK)
#undef BSHMEM_DEV_COLL_WARP
#undef BSHMEM_DEV_COLL_BLOCK
#undef BSHMEM_DEV_COLL_SCOPED

#define BSHMEM_DEV_REDUCE_OP(N, T, OPNAME, OPENUM)                                                                                       \
  BSHMEM_DEV(int, nvshmem_##N##_##OPNAME##_reduce, (nvshmem_team_t team, T* d, const T* s, size_t n), { return bshmem::allreduce<T, OPENUM, bshmem::SCOPE_THREAD>(team, d, s, n); }) \
  BSHMEM_DEV(int, nvshmem_##N##_##OPNAME##_reducescatter, (nvshmem_team_t team, T* d, const T* s, size_t n), { return bshmem::reducescatter<T, OPENUM, bshmem::SCOPE_THREAD>(team, d, s, n); }) \
  BSHMEM_DEVX int nvshmemx_##N##_##OPNAME##_reduce_warp(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::allreduce<T, OPENUM, bshmem::SCOPE_WARP>(team, d, s, n); } \
  BSHMEM_DEVX int nvshmemx_##N##_##OPNAME##_reduce_block(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::allreduce<T, OPENUM, bshmem::SCOPE_BLOCK>(team, d, s, n); } \
  BSHMEM_DEVX int nvshmemx_##N##_##OPNAME##_reducescatter_warp(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::reducescatter<T, OPENUM, bshmem::SCOPE_WARP>(team, d, s, n); } \
  BSHMEM_DEVX int nvshmemx_##N##_##OPNAME##_reducescatter_block(nvshmem_team_t team, T* d, const T* s, size_t n) { return bshmem::reducescatter<T, OPENUM, bshmem::SCOPE_BLOCK>(team, d, s, n); }
#define BSHMEM_DEV_BITWISE(N, T) BSHMEM_DEV_REDUCE_OP(N, T, and, bshmem::OP_AND) BSHMEM_DEV_REDUCE_OP(N, T, or, bshmem::OP_OR) BSHMEM_DEV_REDUCE_OP(N, T, xor, bshmem::OP_XOR)
#define BSHMEM_DEV_ARITH(N, T) BSHMEM_DEV_REDUCE_OP(N, T, min, bshmem::OP_MIN) BSHMEM_DEV_REDUCE_OP(N, T, max, bshmem::OP_MAX) BSHMEM_DEV_REDUCE_OP(N, T, sum, bshmem::OP_SUM) BSHMEM_DEV_REDUCE_OP(N, T, prod, bshmem::OP_PROD)
BSHMEM_BITWISE_REDUCE_TYPES(BSHMEM_DEV_BITWISE)
BSHMEM_STANDARD_REDUCE_TYPES(BSHMEM_DEV_ARITH)
#undef BSHMEM_DEV_BITWISE
#undef BSHMEM_DEV_ARITH
#undef BSHMEM_DEV_REDUCE_OP
BSHMEM_DEVX int nvshmemx_double2_maxloc_reduce_block(nvshmem_team_t team, double2* d, const double2* s, size_t n) {
  return n == 1 ? bshmem::maxloc_double2<bshmem::SCOPE_BLOCK>(team, d, s) : 1;
}

// ------------------------------------------------------------------ byte collectives at warp / block scope
BSHMEM_DEVX int nvshmemx_alltoallmem_warp(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return bshmem::alltoall<char, bshmem::SCOPE_WARP>(team, (char*)d, (const char*)s, bytes); }
BSHMEM_DEVX int nvshmemx_alltoallmem_block(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return bshmem::alltoall<char, bshmem::SCOPE_BLOCK>(team, (char*)d, (const char*)s, bytes); }
BSHMEM_DEVX int nvshmemx_fcollectmem_warp(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return bshmem::fcollect<char, bshmem::SCOPE_WARP>(team, (char*)d, (const char*)s, bytes); }
BSHMEM_DEVX int nvshmemx_fcollectmem_block(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return bshmem::fcollect<char, bshmem::SCOPE_BLOCK>(team, (char*)d, (const char*)s, bytes); }
BSHMEM_DEVX int nvshmemx_broadcastmem_warp(nvshmem_team_t team, void* d, const void* s, size_t bytes, int root) { return bshmem::broadcast<char, bshmem::SCOPE_WARP>(team, (char*)d, (const char*)s, bytes, root); }
BSHMEM_DEVX int nvshmemx_broadcastmem_block(nvshmem_team_t team, void* d, const void* s, size_t bytes, int root) { return bshmem::broadcast<char, bshmem::SCOPE_BLOCK>(team, (char*)d, (const char*)s, bytes, root); }

// ------------------------------------------------------------------ sized strided and signalling variants at warp / block scope
#define BSHMEM_DEV_SIZED_MORE(BITS, T)                                                                                                   \
  BSHMEM_DEVX void nvshmemx_iput##BITS##_warp(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iput<T, bshmem::SCOPE_WARP>((T*)d, (const T*)s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmemx_iput##BITS##_block(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iput<T, bshmem::SCOPE_BLOCK>((T*)d, (const T*)s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmemx_iget##BITS##_warp(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iget<T, bshmem::SCOPE_WARP>((T*)d, (const T*)s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmemx_iget##BITS##_block(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { bshmem::iget<T, bshmem::SCOPE_BLOCK>((T*)d, (const T*)s, dst, sst, n, pe); } \
  BSHMEM_DEVX void nvshmem_put##BITS##_signal_nbi(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * (BITS / 8), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_signal_nbi_warp(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_WARP>(d, s, n * (BITS / 8), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_put##BITS##_signal_nbi_block(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { bshmem::putmem_signal<bshmem::SCOPE_BLOCK>(d, s, n * (BITS / 8), sig, v, op, pe); }
BSHMEM_SIZES(BSHMEM_DEV_SIZED_MORE)
#undef BSHMEM_DEV_SIZED_MORE

// ------------------------------------------------------------------ queue-pair variants
// On transports with queue pairs the caller may pick the one an operation travels on.  Peers here are reached with
// plain loads and stores over NVLink, which have no queues: the handle is accepted and ignored, and quiet / fence on
// a set of queue pairs are quiet / fence.  (reference: src/include/host/nvshmemx_api.h, "QPair (qp) device APIs")
#define BSHMEM_DEV_QP(N, T)                                                                                                              \
  BSHMEM_DEVX void nvshmemx_qp_##N##_p(T* d, const T v, int pe, nvshmemx_qp_handle_t) { bshmem::p<T>(d, v, pe); }                         \
  BSHMEM_DEVX T nvshmemx_qp_##N##_g(const T* s, int pe, nvshmemx_qp_handle_t) { return bshmem::g<T>(s, pe); }                             \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::putmem<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_get(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::getmem<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_nbi(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_get_nbi(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::getmem_nbi<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_signal(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_signal_nbi(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_signal<bshmem::SCOPE_THREAD>(d, s, n * sizeof(T), sig, v, op, pe); }
BSHMEM_RMA_TYPES(BSHMEM_DEV_QP)
#undef BSHMEM_DEV_QP
#define BSHMEM_DEV_QP_SCOPED(N, T, SUF, SC)                                                                                              \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_##SUF(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::putmem<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_get_##SUF(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::getmem<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_nbi_##SUF(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_nbi<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_get_nbi_##SUF(T* d, const T* s, size_t n, int pe, nvshmemx_qp_handle_t) { bshmem::getmem_nbi<SC>(d, s, n * sizeof(T), pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_signal_##SUF(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_signal<SC>(d, s, n * sizeof(T), sig, v, op, pe); } \
  BSHMEM_DEVX void nvshmemx_qp_##N##_put_signal_nbi_##SUF(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, nvshmemx_qp_handle_t) { bshmem::putmem_signal<SC>(d, s, n * sizeof(T), sig, v, op, pe); }
#define BSHMEM_DEV_QP_WARP(N, T) BSHMEM_DEV_QP_SCOPED(N, T, warp, bshmem::SCOPE_WARP)
#define BSHMEM_DEV_QP_BLOCK(N, T) BSHMEM_DEV_QP_SCOPED(N, T, block, bshmem::SCOPE_BLOCK)
BSHMEM_RMA_TYPES(BSHMEM_DEV_QP_WARP)
BSHMEM_RMA_TYPES(BSHMEM_DEV_QP_BLOCK)
#undef BSHMEM_DEV_QP_WARP
#undef BSHMEM_DEV_QP_BLOCK
#undef BSHMEM_DEV_QP_SCOPED
BSHMEM_DEVX void nvshmemx_qp_signal_op(uint64_t* sig, uint64_t v, int op, int pe, nvshmemx_qp_handle_t) { bshmem::signal_op(sig, v, op, pe); }
BSHMEM_DEVX void nvshmemx_qp_quiet(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }
BSHMEM_DEVX void nvshmemx_qp_quiet_warp(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }
BSHMEM_DEVX void nvshmemx_qp_quiet_block(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }
BSHMEM_DEVX void nvshmemx_qp_fence(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }
BSHMEM_DEVX void nvshmemx_qp_fence_warp(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }
BSHMEM_DEVX void nvshmemx_qp_fence_block(int, nvshmemx_qp_handle_t*, int) { bshmem::fence_sys(); }

#undef BSHMEM_DEV
#undef BSHMEM_DEVX
