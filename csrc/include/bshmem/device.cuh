// Device-side one-sided core for sm_100a: address translation, put/get/p/g,
// signals, ordering, bounded waits and atomics, for thread, warp, warpgroup and
// block scope.  Header only; every CUDA module that includes it carries its own
// `__constant__` copy of the state, which a static registrar announces to the
// host library so that the host can fill it.
//
// All peers are load/store reachable (one NVSwitch domain), so every operation
// is a handful of instructions issued by the calling threads:
//   data     : 16-byte vector ld/st on the translated address
//   signals  : st.release.sys / red.release.sys.add, read with ld.acquire.sys
//   ordering : fence.acq_rel.sys (quiet and fence coincide on a load/store fabric)
//   atomics  : atom.sys on the translated address
// Every spin is bounded by `wait_timeout_ns`; on expiry the wait records what it
// was waiting for in the host-visible status block and RETURNS non-zero.  Nothing
// here traps or spins for ever
// (reference behaviour: src/include/non_abi/device/common/nvshmemi_common_device.cuh,
//  src/include/non_abi/device/wait/nvshmemi_wait_until_apis.cuh, src/include/device/nvshmem_defines.h).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "state.h"

// Where the device-side copy of the state lives:
//   default               one `static __constant__` copy per translation unit, announced to the host library by a
//                         static registrar (no relocatable device code, nothing for the user to do);
//   BSHMEM_DEVICE_MODULE  for device code that is compiled on its own (nvcc -cubin / -fatbin / -ptx) and loaded with
//                         the driver API: the copy gets the unmangled global name `bshmemi_state_d`, which
//                         nvshmemx_cumodule_init / nvshmemx_culibrary_init look up in the loaded module and fill.
//                         Define it in ONE translation unit of such a module (with -rdc the others declare it extern).
#if defined(BSHMEM_DEVICE_MODULE)
extern "C" {
__constant__ bshmemi_state_t bshmemi_state_d;
}
#else
#ifndef BSHMEM_STATE_LINKAGE
#define BSHMEM_STATE_LINKAGE static
#endif
BSHMEM_STATE_LINKAGE __constant__ bshmemi_state_t bshmemi_state_d;
#endif

extern "C" void bshmemi_register_module(void* (*getter)(), const char* name);

#if !defined(BSHMEM_DEVICE_MODULE)
namespace bshmem_detail {
static void* state_symbol_address() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, bshmemi_state_d) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return p;
}
struct ModuleRegistrar {
  ModuleRegistrar() { bshmemi_register_module(&state_symbol_address, __FILE__); }
};
static ModuleRegistrar module_registrar_instance;
}  // namespace bshmem_detail
#endif

namespace bshmem {

enum Scope { SCOPE_THREAD = 0, SCOPE_WARP = 1, SCOPE_WARPGROUP = 2, SCOPE_BLOCK = 3 };
enum Cmp { CMP_EQ = 0, CMP_NE = 1, CMP_GT = 2, CMP_LE = 3, CMP_LT = 4, CMP_GE = 5 };
enum SignalOp { SIGNAL_SET = 9, SIGNAL_ADD = 10 };

// ------------------------------------------------------------------ scopes
template <int SCOPE>
__device__ __forceinline__ int group_rank() {
  if (SCOPE == SCOPE_THREAD) return 0;
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  if (SCOPE == SCOPE_WARP) return tid & 31;
  if (SCOPE == SCOPE_WARPGROUP) return tid & 127;
  return tid;
}
template <int SCOPE>
__device__ __forceinline__ int group_size() {
  if (SCOPE == SCOPE_THREAD) return 1;
  if (SCOPE == SCOPE_WARP) return 32;
  if (SCOPE == SCOPE_WARPGROUP) return 128;
  return blockDim.x * blockDim.y * blockDim.z;
}
template <int SCOPE>
__device__ __forceinline__ void group_sync() {
  if (SCOPE == SCOPE_WARP) __syncwarp();
  else if (SCOPE == SCOPE_WARPGROUP) {
    // Named barrier 1 + warpgroup index: barrier 0 stays with __syncthreads.
    const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
    asm volatile("bar.sync %0, 128;" ::"r"(1 + (tid >> 7)) : "memory");
  } else if (SCOPE == SCOPE_BLOCK) __syncthreads();
}

// ------------------------------------------------------------------ raw memory operations
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ------------------------------------------------------------------ state access
__device__ __forceinline__ int my_pe() { return bshmemi_state_d.mype; }
__device__ __forceinline__ int n_pes() { return bshmemi_state_d.npes; }
__device__ __forceinline__ bshmemi_status_t* status_block() { return (bshmemi_status_t*)bshmemi_state_d.status; }
__device__ __forceinline__ void report_error(uint32_t bits) {
  bshmemi_status_t* s = status_block();
  if (s) atomicOr_system((unsigned int*)&s->error_bits, bits);
}
__device__ __forceinline__ uint32_t error_bits() {
  bshmemi_status_t* s = status_block();
  return s ? s->error_bits : 0u;
}

// Address of the same symmetric object on PE `pe`: one multiply-add, no table.
template <class T>
__device__ __forceinline__ T* translate(const T* p, int pe) {
  const int64_t delta = (int64_t)(pe - bshmemi_state_d.mype) * (int64_t)bshmemi_state_d.heap_stride;
  return (T*)((char*)p + delta);
}
__device__ __forceinline__ bool in_heap(const void* p) {
  const uint64_t a = (uint64_t)p;
  return a >= bshmemi_state_d.heap_base && a < bshmemi_state_d.heap_base + bshmemi_state_d.heap_size;
}
// nvshmem_ptr: null for a non-symmetric address or an invalid PE.
__device__ __forceinline__ void* ptr(const void* p, int pe) {
  if (!in_heap(p) || pe < 0 || pe >= bshmemi_state_d.npes) return nullptr;
  return translate((const char*)p, pe);
}
// Multicast alias of a symmetric address (world team), or null without NVLS.
__device__ __forceinline__ void* mc_ptr(const void* p) {
  if (!bshmemi_state_d.mc_base || !in_heap(p)) return nullptr;
  return (void*)(bshmemi_state_d.mc_base + ((uint64_t)p - bshmemi_state_d.heap_base));
}
// Debug-build style check used by the data paths when NVSHMEM_ENABLE_ERROR_CHECKS
// is set: records the fault and tells the caller to skip the access.
__device__ __forceinline__ bool check_target(const void* sym, int pe) {
  if (!bshmemi_state_d.debug_checks) return true;
  if (pe < 0 || pe >= bshmemi_state_d.npes) { report_error(BSHMEM_ERR_BAD_PE); return false; }
  if (!in_heap(sym)) { report_error(BSHMEM_ERR_BAD_ADDRESS); return false; }
  return true;
}

// ------------------------------------------------------------------ group memcpy
// Picks the widest vector both addresses and the length allow (16/8/4/2/1 bytes);
// thread i of the group moves elements i, i+G, i+2G, … so that a warp's accesses
// are contiguous.  The 16-byte loop is unrolled 4x to keep several NVLink
// transactions in flight per thread.
template <int SCOPE>
__device__ __forceinline__ void memcpy_group(void* __restrict__ dst, const void* __restrict__ src, size_t bytes) {
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const uintptr_t d = (uintptr_t)dst, s = (uintptr_t)src;
  size_t done = 0;
  if (((d | s) & 15) == 0 && bytes >= 16) {
    const size_t n = bytes / 16;
    uint4* __restrict__ D = (uint4*)dst;
    const uint4* __restrict__ S = (const uint4*)src;
    size_t i = rank;
    for (; i + 3 * (size_t)G < n; i += 4 * (size_t)G) {
      uint4 a = S[i], b = S[i + G], c = S[i + 2 * (size_t)G], e = S[i + 3 * (size_t)G];
      D[i] = a; D[i + G] = b; D[i + 2 * (size_t)G] = c; D[i + 3 * (size_t)G] = e;
    }
    for (; i < n; i += G) D[i] = S[i];
    done = n * 16;
  } else if (((d | s) & 7) == 0 && bytes >= 8) {
    const size_t n = bytes / 8;
    for (size_t i = rank; i < n; i += G) ((uint64_t*)dst)[i] = ((const uint64_t*)src)[i];
    done = n * 8;
  } else if (((d | s) & 3) == 0 && bytes >= 4) {
    const size_t n = bytes / 4;
    for (size_t i = rank; i < n; i += G) ((uint32_t*)dst)[i] = ((const uint32_t*)src)[i];
    done = n * 4;
  } else if (((d | s) & 1) == 0 && bytes >= 2) {
    const size_t n = bytes / 2;
    for (size_t i = rank; i < n; i += G) ((uint16_t*)dst)[i] = ((const uint16_t*)src)[i];
    done = n * 2;
  }
  for (size_t i = done + rank; i < bytes; i += G) ((char*)dst)[i] = ((const char*)src)[i];
}

// ------------------------------------------------------------------ ordering
// On a pure load/store fabric quiet and fence are the same instruction: a
// system-scope fence by one thread of the group (the others' writes are ordered
// before it by the group barrier).
template <int SCOPE>
__device__ __forceinline__ void quiet() {
  group_sync<SCOPE>();
  if (group_rank<SCOPE>() == 0) fence_sys();
  group_sync<SCOPE>();
}
template <int SCOPE>
__device__ __forceinline__ void fence() { quiet<SCOPE>(); }

// ------------------------------------------------------------------ RMA
template <class T>
__device__ __forceinline__ void p(T* dest, T value, int pe) {
  if (!check_target(dest, pe)) return;
  *(volatile T*)translate(dest, pe) = value;
}
template <class T>
__device__ __forceinline__ T g(const T* src, int pe) {
  if (!check_target(src, pe)) return T();
  return *(const volatile T*)translate(src, pe);
}
// Non-blocking put: the copy is issued; completion needs quiet().
template <int SCOPE>
__device__ __forceinline__ void putmem_nbi(void* dest, const void* src, size_t bytes, int pe) {
  if (!check_target(dest, pe)) return;
  memcpy_group<SCOPE>(translate((char*)dest, pe), src, bytes);
}
// Blocking put: on return the source may be reused by any thread of the group.
template <int SCOPE>
__device__ __forceinline__ void putmem(void* dest, const void* src, size_t bytes, int pe) {
  putmem_nbi<SCOPE>(dest, src, bytes, pe);
  group_sync<SCOPE>();
}
template <int SCOPE>
__device__ __forceinline__ void getmem_nbi(void* dest, const void* src, size_t bytes, int pe) {
  if (!check_target(src, pe)) return;
  memcpy_group<SCOPE>(dest, translate((const char*)src, pe), bytes);
}
template <int SCOPE>
__device__ __forceinline__ void getmem(void* dest, const void* src, size_t bytes, int pe) {
  getmem_nbi<SCOPE>(dest, src, bytes, pe);
  group_sync<SCOPE>();
}
// Strided put/get: element strides `dst`/`sst`, `nelems` elements.
template <class T, int SCOPE>
__device__ __forceinline__ void iput(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe) {
  if (!check_target(dest, pe)) return;
  T* d = translate(dest, pe);
  for (size_t i = group_rank<SCOPE>(); i < nelems; i += group_size<SCOPE>()) d[i * dst] = src[i * sst];
  group_sync<SCOPE>();
}
template <class T, int SCOPE>
__device__ __forceinline__ void iget(T* dest, const T* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe) {
  if (!check_target(src, pe)) return;
  const T* s = translate(src, pe);
  for (size_t i = group_rank<SCOPE>(); i < nelems; i += group_size<SCOPE>()) dest[i * dst] = s[i * sst];
  group_sync<SCOPE>();
}

// ------------------------------------------------------------------ signals
// Bare signal update: an atomic store or add with no ordering of its own.  Code that publishes
// data with it orders the data first (fence / quiet); putmem_signal below does so itself.
__device__ __forceinline__ void signal_op(uint64_t* sig_addr, uint64_t value, int op, int pe) {
  uint64_t* remote = translate(sig_addr, pe);
  if (op == SIGNAL_ADD) asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(remote), "l"(value) : "memory");
  else st_relaxed_sys(remote, value);
}
__device__ __forceinline__ void signal_op_release(uint64_t* sig_addr, uint64_t value, int op, int pe) {
  uint64_t* remote = translate(sig_addr, pe);
  if (op == SIGNAL_ADD) red_add_release_sys(remote, value);
  else st_release_sys(remote, value);
}
// Copy, then one thread publishes the signal with release semantics: a peer that
// acquires the signal value sees the whole payload.
template <int SCOPE>
__device__ __forceinline__ void putmem_signal(void* dest, const void* src, size_t bytes, uint64_t* sig_addr, uint64_t value, int op, int pe) {
  if (!check_target(dest, pe)) return;
  memcpy_group<SCOPE>(translate((char*)dest, pe), src, bytes);
  group_sync<SCOPE>();
  if (group_rank<SCOPE>() == 0) signal_op_release(sig_addr, value, op, pe);  // release: cumulative over the group's stores (ordered here by the barrier)
}
__device__ __forceinline__ uint64_t signal_fetch(const uint64_t* sig_addr) { return ld_acquire_sys(sig_addr); }

// ------------------------------------------------------------------ bounded waits
template <class T>
__device__ __forceinline__ bool compare(T found, int cmp, T want) {
  switch (cmp) {
    case CMP_EQ: return found == want;
    case CMP_NE: return found != want;
    case CMP_GT: return found > want;
    case CMP_LE: return found <= want;
    case CMP_LT: return found < want;
    default: return found >= want;
  }
}
__device__ __forceinline__ void record_timeout(const void* addr, uint64_t expected, uint64_t found, uint32_t where) {
  bshmemi_status_t* s = status_block();
  if (!s) return;
  if (atomicAdd_system((unsigned int*)&s->timeout_count, 1u) == 0) {
    s->timeout_addr = (uint64_t)addr;
    s->timeout_expected = expected;
    s->timeout_found = found;
    s->timeout_where = where;
  }
  __threadfence_system();
  atomicOr_system((unsigned int*)&s->error_bits, BSHMEM_ERR_WAIT_TIMEOUT);
}
// One polling read with acquire semantics at system scope: 32- and 64-bit words use ld.acquire.sys
// (no separate fence is then needed once the comparison holds); narrower types use a volatile load
// and the caller fences.
template <class T>
__device__ __forceinline__ T poll_load(const T* p, bool* needs_fence) {
  if (sizeof(T) == 8) {
    uint64_t v = ld_acquire_sys((const uint64_t*)p);
    T out;
    memcpy(&out, &v, 8);
    return out;
  } else if (sizeof(T) == 4) {
    uint32_t v = ld_acquire_sys((const uint32_t*)p);
    T out;
    memcpy(&out, &v, 4);
    return out;
  }
  *needs_fence = true;
  return *(const volatile T*)p;
}
// Polls until cmp(*ivar, value) holds.  Returns 0 on success, 1 after `wait_timeout_ns`
// (the time-out is recorded; the caller carries on).  Data published before the flag is
// visible to the caller on return.
template <class T>
__device__ __forceinline__ int wait_until(const T* ivar, int cmp, T value, uint32_t where = BSHMEM_WHERE_WAIT_UNTIL) {
  bool needs_fence = false;
  T found = poll_load(ivar, &needs_fence);
  if (!compare(found, cmp, value)) {
    const uint64_t start = global_timer_ns(), limit = bshmemi_state_d.wait_timeout_ns;
    uint32_t spins = 0;
    for (;;) {
      found = poll_load(ivar, &needs_fence);
      if (compare(found, cmp, value)) break;
      if ((++spins & 0x3ff) == 0) {
        if (global_timer_ns() - start > limit) {
          record_timeout((const void*)ivar, (uint64_t)value, (uint64_t)found, where);
          return 1;
        }
      }
    }
  }
  if (needs_fence) fence_sys();
  return 0;
}
__device__ __forceinline__ int wait_ge_u64(const uint64_t* ivar, uint64_t value, uint32_t where) {
  return wait_until<uint64_t>(ivar, CMP_GE, value, where);
}
template <class T>
__device__ __forceinline__ int test(const T* ivar, int cmp, T value) {
  bool needs_fence = false;
  T found = poll_load(ivar, &needs_fence);
  if (!compare(found, cmp, value)) return 0;
  if (needs_fence) fence_sys();
  return 1;
}
// wait_until_all / any / some and their _vector forms.  `status[i] != 0` excludes entry i.
template <class T>
__device__ __forceinline__ int wait_until_all(const T* ivars, size_t n, const int* status, int cmp, const T* values, T value) {
  int err = 0;
  for (size_t i = 0; i < n; ++i)
    if (!status || !status[i]) err |= wait_until(ivars + i, cmp, values ? values[i] : value);
  return err;
}
template <class T>
__device__ __forceinline__ size_t wait_until_any(const T* ivars, size_t n, const int* status, int cmp, const T* values, T value) {
  bool candidates = false;
  for (size_t i = 0; i < n; ++i) candidates |= !status || !status[i];
  if (!candidates) return (size_t)-1;
  const uint64_t start = global_timer_ns(), limit = bshmemi_state_d.wait_timeout_ns;
  for (;;) {
    for (size_t i = 0; i < n; ++i)
      if ((!status || !status[i]) && test(ivars + i, cmp, values ? values[i] : value)) return i;
    if (global_timer_ns() - start > limit) {
      record_timeout(ivars, 0, 0, BSHMEM_WHERE_WAIT_UNTIL);
      return (size_t)-1;
    }
  }
}
template <class T>
__device__ __forceinline__ size_t wait_until_some(const T* ivars, size_t n, size_t* indices, const int* status, int cmp, const T* values, T value) {
  size_t first = wait_until_any(ivars, n, status, cmp, values, value);
  if (first == (size_t)-1) return 0;
  size_t count = 0;
  for (size_t i = 0; i < n; ++i)
    if ((!status || !status[i]) && test(ivars + i, cmp, values ? values[i] : value)) indices[count++] = i;
  return count;
}
template <class T>
__device__ __forceinline__ int test_all(const T* ivars, size_t n, const int* status, int cmp, const T* values, T value) {
  for (size_t i = 0; i < n; ++i)
    if ((!status || !status[i]) && !test(ivars + i, cmp, values ? values[i] : value)) return 0;
  return 1;
}
template <class T>
__device__ __forceinline__ size_t test_any(const T* ivars, size_t n, const int* status, int cmp, const T* values, T value) {
  for (size_t i = 0; i < n; ++i)
    if ((!status || !status[i]) && test(ivars + i, cmp, values ? values[i] : value)) return i;
  return (size_t)-1;
}
template <class T>
__device__ __forceinline__ size_t test_some(const T* ivars, size_t n, size_t* indices, const int* status, int cmp, const T* values, T value) {
  size_t count = 0;
  for (size_t i = 0; i < n; ++i)
    if ((!status || !status[i]) && test(ivars + i, cmp, values ? values[i] : value)) indices[count++] = i;
  return count;
}

// ------------------------------------------------------------------ atomics
// One atom.sys on the translated address.  32- and 64-bit integers map onto the
// unsigned hardware atomics; float/double swap and fetch go through their bits.
template <class T, class U>
__device__ __forceinline__ U as_bits(T v) {
  static_assert(sizeof(T) == sizeof(U), "size mismatch");
  U u;
  memcpy(&u, &v, sizeof(U));
  return u;
}
template <class T>
struct AmoWord { typedef unsigned int type; };
template <> struct AmoWord<long> { typedef unsigned long long type; };
template <> struct AmoWord<unsigned long> { typedef unsigned long long type; };
template <> struct AmoWord<long long> { typedef unsigned long long type; };
template <> struct AmoWord<unsigned long long> { typedef unsigned long long type; };
template <> struct AmoWord<double> { typedef unsigned long long type; };

template <class T>
__device__ __forceinline__ T atomic_fetch_add(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  W old = atomicAdd_system((W*)translate(target, pe), as_bits<T, W>(value));
  return as_bits<W, T>(old);
}
template <class T>
__device__ __forceinline__ void atomic_add(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  W* a = (W*)translate(target, pe);
  if (sizeof(W) == 8) asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(a), "l"((unsigned long long)as_bits<T, W>(value)) : "memory");
  else asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(a), "r"((unsigned int)as_bits<T, W>(value)) : "memory");
}
template <class T>
__device__ __forceinline__ T atomic_compare_swap(T* target, T cond, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicCAS_system((W*)translate(target, pe), as_bits<T, W>(cond), as_bits<T, W>(value)));
}
template <class T>
__device__ __forceinline__ T atomic_swap(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicExch_system((W*)translate(target, pe), as_bits<T, W>(value)));
}
template <class T>
__device__ __forceinline__ T atomic_fetch(const T* target, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicOr_system((W*)translate(target, pe), (W)0));
}
template <class T>
__device__ __forceinline__ void atomic_set(T* target, T value, int pe) { (void)atomic_swap(target, value, pe); }
template <class T>
__device__ __forceinline__ T atomic_fetch_and(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicAnd_system((W*)translate(target, pe), as_bits<T, W>(value)));
}
template <class T>
__device__ __forceinline__ T atomic_fetch_or(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicOr_system((W*)translate(target, pe), as_bits<T, W>(value)));
}
template <class T>
__device__ __forceinline__ T atomic_fetch_xor(T* target, T value, int pe) {
  typedef typename AmoWord<T>::type W;
  return as_bits<W, T>(atomicXor_system((W*)translate(target, pe), as_bits<T, W>(value)));
}

// Device-side global exit: raises the request for the host watchdog and returns;
// the kernel is expected to finish normally (no endless spin on the device).
__device__ __forceinline__ void global_exit(int status) {
  bshmemi_status_t* s = status_block();
  if (!s) return;
  s->global_exit_code = status;
  __threadfence_system();
  s->global_exit_req = 1;
  atomicOr_system((unsigned int*)&s->error_bits, BSHMEM_ERR_GLOBAL_EXIT);
}

}  // namespace bshmem
