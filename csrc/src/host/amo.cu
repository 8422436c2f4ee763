#include <string.h>

#include "../../include/bshmem/device.cuh"
#include "../state/runtime.h"
#include "../util/log.h"
#include "amo.h"

namespace bshmem {

template <class W>
__device__ W amo_apply(int op, W* addr, W value, W cond) {
  switch (op) {
    case AMO_ADD:
    case AMO_FETCH_ADD: return atomicAdd_system(addr, value);
    case AMO_CAS: return atomicCAS_system(addr, cond, value);
    case AMO_SWAP: return atomicExch_system(addr, value);
    case AMO_AND: return atomicAnd_system(addr, value);
    case AMO_OR: return atomicOr_system(addr, value);
    case AMO_XOR: return atomicXor_system(addr, value);
    default: return atomicOr_system(addr, (W)0);
  }
}

__global__ void amo_kernel(int op, void* target, unsigned long long value, unsigned long long cond, int width, int pe, unsigned long long* old) {
  unsigned long long result;
  if (width == 8) result = amo_apply<unsigned long long>(op, (unsigned long long*)translate((char*)target, pe), value, cond);
  else result = amo_apply<unsigned int>(op, (unsigned int*)translate((char*)target, pe), (unsigned int)value, (unsigned int)cond);
  if (old) *old = result;
}

template <class W>
static W host_apply(int op, W* addr, W value, W cond) {
  switch (op) {
    case AMO_ADD:
    case AMO_FETCH_ADD: return __atomic_fetch_add(addr, value, __ATOMIC_ACQ_REL);
    case AMO_CAS: {
      W expected = cond;
      __atomic_compare_exchange_n(addr, &expected, value, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
      return expected;
    }
    case AMO_SWAP: return __atomic_exchange_n(addr, value, __ATOMIC_ACQ_REL);
    case AMO_AND: return __atomic_fetch_and(addr, value, __ATOMIC_ACQ_REL);
    case AMO_OR: return __atomic_fetch_or(addr, value, __ATOMIC_ACQ_REL);
    case AMO_XOR: return __atomic_fetch_xor(addr, value, __ATOMIC_ACQ_REL);
    default: return __atomic_load_n(addr, __ATOMIC_ACQUIRE);
  }
}

int host_amo(int op, void* target, const void* value, const void* cond, size_t width, int pe, void* old) {
  Runtime& r = rt();
  if (!is_initialized() || (width != 4 && width != 8)) return ST_INVALID_VALUE;
  void* remote = r.heap->translate(target, pe);
  if (!remote) {
    ERROR_PRINT("atomic: %p is not a symmetric address or PE %d is out of range", target, pe);
    return ST_INVALID_VALUE;
  }
  unsigned long long v = 0, c = 0, result = 0;
  if (value) memcpy(&v, value, width);
  if (cond) memcpy(&c, cond, width);
  if (!r.have_gpu) {
    if (width == 8) result = host_apply<unsigned long long>(op, (unsigned long long*)remote, v, c);
    else result = host_apply<unsigned int>(op, (unsigned int*)remote, (unsigned int)v, (unsigned int)c);
  } else {
    static unsigned long long* pinned = nullptr;
    if (!pinned && cudaHostAlloc((void**)&pinned, sizeof(*pinned), cudaHostAllocMapped) != cudaSuccess) return ST_OUT_OF_MEMORY;
    unsigned long long* dev_view = nullptr;
    cudaHostGetDevicePointer((void**)&dev_view, pinned, 0);
    amo_kernel<<<1, 1, 0, r.stream>>>(op, target, v, c, (int)width, pe, dev_view);
    if (cudaStreamSynchronize(r.stream) != cudaSuccess) return ST_INTERNAL;
    result = *pinned;
  }
  if (old) memcpy(old, &result, width);
  return ST_SUCCESS;
}

}  // namespace bshmem
