// NVLink multicast (NVLS) instructions for sm_100a.  A `multimem` address is
// the multicast alias of a symmetric address (bshmem::mc_ptr): a store reaches
// the same offset of every PE's heap, a `ld_reduce` returns the element-wise
// reduction over all PEs' copies, performed inside the NVSwitch.  All accesses
// of floating types are 16 bytes wide, 16-bit types accumulate in fp32 (.acc::f32); integer
// reductions (add, min, max, and, or, xor) are one 32- or 64-bit element per instruction
// (reference: src/include/non_abi/device/coll/reduce.cuh:124-223,
//  src/include/non_abi/device/common/nvshmemi_common_device.cuh:156-252).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

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

// Integer reductions inside the switch: one element of 4 or 8 bytes per instruction.  `OP` uses the numbering of
// the collectives (0 and, 1 or, 2 xor, 3 min, 4 max, 5 sum).  Signedness matters for min / max only; add and the
// bitwise operators work on the bit pattern (reference: src/include/non_abi/device/coll/reducescatter.cuh:91-200).
#define BSHMEM_MM_INT(NAME, OPSTR, TYPESTR, CTYPE, REG)                                                                 \
  __device__ __forceinline__ CTYPE multimem_##NAME(const void* a) {                                                     \
    CTYPE v;                                                                                                            \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." OPSTR "." TYPESTR " %0, [%1];" : "=" REG(v) : "l"(a) : "memory"); \
    return v;                                                                                                           \
  }
BSHMEM_MM_INT(add_u32, "add", "u32", uint32_t, "r")
BSHMEM_MM_INT(add_u64, "add", "u64", uint64_t, "l")
BSHMEM_MM_INT(min_u32, "min", "u32", uint32_t, "r")
BSHMEM_MM_INT(min_s32, "min", "s32", int32_t, "r")
BSHMEM_MM_INT(min_u64, "min", "u64", uint64_t, "l")
BSHMEM_MM_INT(min_s64, "min", "s64", int64_t, "l")
BSHMEM_MM_INT(max_u32, "max", "u32", uint32_t, "r")
BSHMEM_MM_INT(max_s32, "max", "s32", int32_t, "r")
BSHMEM_MM_INT(max_u64, "max", "u64", uint64_t, "l")
BSHMEM_MM_INT(max_s64, "max", "s64", int64_t, "l")
BSHMEM_MM_INT(and_b32, "and", "b32", uint32_t, "r")
BSHMEM_MM_INT(and_b64, "and", "b64", uint64_t, "l")
BSHMEM_MM_INT(or_b32, "or", "b32", uint32_t, "r")
BSHMEM_MM_INT(or_b64, "or", "b64", uint64_t, "l")
BSHMEM_MM_INT(xor_b32, "xor", "b32", uint32_t, "r")
BSHMEM_MM_INT(xor_b64, "xor", "b64", uint64_t, "l")
#undef BSHMEM_MM_INT

// Element-wise reduction of one integer element of type T over all PEs; `supported` says whether the switch can do it.
template <class T, int OP, bool IS_INT = std::is_integral<T>::value, int BYTES = (int)sizeof(T)>
struct MultimemInt {
  static constexpr bool supported = false;
  __device__ static __forceinline__ T ld(const void*) { return T(); }
};
template <class T, int OP>
struct MultimemInt<T, OP, true, 4> {
  static constexpr bool supported = OP >= 0 && OP <= 5;
  __device__ static __forceinline__ T ld(const void* a) {
    constexpr bool sgn = std::is_signed<T>::value;
    uint32_t r;
    if (OP == 0) r = multimem_and_b32(a);
    else if (OP == 1) r = multimem_or_b32(a);
    else if (OP == 2) r = multimem_xor_b32(a);
    else if (OP == 3) r = sgn ? (uint32_t)multimem_min_s32(a) : multimem_min_u32(a);
    else if (OP == 4) r = sgn ? (uint32_t)multimem_max_s32(a) : multimem_max_u32(a);
    else r = multimem_add_u32(a);
    return (T)r;
  }
};
template <class T, int OP>
struct MultimemInt<T, OP, true, 8> {
  static constexpr bool supported = OP >= 0 && OP <= 5;
  __device__ static __forceinline__ T ld(const void* a) {
    constexpr bool sgn = std::is_signed<T>::value;
    uint64_t r;
    if (OP == 0) r = multimem_and_b64(a);
    else if (OP == 1) r = multimem_or_b64(a);
    else if (OP == 2) r = multimem_xor_b64(a);
    else if (OP == 3) r = sgn ? (uint64_t)multimem_min_s64(a) : multimem_min_u64(a);
    else if (OP == 4) r = sgn ? (uint64_t)multimem_max_s64(a) : multimem_max_u64(a);
    else r = multimem_add_u64(a);
    return (T)r;
  }
};

// What the switch can reduce for element type T and operator OP, and in pieces of how many bytes: sums of
// float / half / bfloat16 as 16-byte vectors, the integer operators one element at a time.
template <class T, int OP>
struct NvlsReduce {
  static constexpr bool vector16 = OP == 5 && MultimemSum<T>::supported;
  static constexpr bool scalar = !vector16 && MultimemInt<T, OP>::supported;
  static constexpr bool supported = vector16 || scalar;
  static constexpr int grain = vector16 ? 16 : (int)sizeof(T);
};

}  // namespace bshmem
