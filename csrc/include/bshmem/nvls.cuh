// NVLink multicast (NVLS) instructions for sm_100a.  A `multimem` address is
// the multicast alias of a symmetric address (bshmem::mc_ptr): a store reaches
// the same offset of every PE's heap, a `ld_reduce` returns the element-wise
// reduction over all PEs' copies, performed inside the NVSwitch.  All accesses
// are 16 bytes wide; 16-bit types accumulate in fp32 (.acc::f32)
// (reference: src/include/non_abi/device/coll/reduce.cuh:124-223,
//  src/include/non_abi/device/common/nvshmemi_common_device.cuh:156-252).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace bshmem {

__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_u64(void* mc_addr, uint64_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_addr), "l"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_u32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add_u64(void* mc_addr, uint64_t v) {
  asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(mc_addr), "l"(v) : "memory");
}

// Sum over all PEs of the 16 bytes at `mc_addr`, by element type.
template <class T>
struct MultimemSum;
template <>
struct MultimemSum<float> {
  static constexpr bool supported = true;
  __device__ static __forceinline__ uint4 ld(const void* a) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a) : "memory");
    return v;
  }
};
template <>
struct MultimemSum<__half> {
  static constexpr bool supported = true;
  __device__ static __forceinline__ uint4 ld(const void* a) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a) : "memory");
    return v;
  }
};
template <>
struct MultimemSum<__nv_bfloat16> {
  static constexpr bool supported = true;
  __device__ static __forceinline__ uint4 ld(const void* a) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a) : "memory");
    return v;
  }
};
template <class T>
struct MultimemSum {
  static constexpr bool supported = false;
  __device__ static __forceinline__ uint4 ld(const void*) { return make_uint4(0, 0, 0, 0); }
};

}  // namespace bshmem
