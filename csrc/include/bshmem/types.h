// Type tables of the public API.  Each row is X(api_name, c_type); the API
// generators expand them into the nvshmem_<api_name>_* functions.  The names are
// part of the OpenSHMEM / NVSHMEM interface
// (reference: src/include/device_host/nvshmem_common.cuh:48-200, src/include/host/nvshmem_api.h:93-195).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>

// clang-format off
#define BSHMEM_RMA_TYPES(X)                                                                         \
  X(bfloat16, __nv_bfloat16) X(half, half) X(float, float) X(double, double) X(char, char)          \
  X(short, short) X(schar, signed char) X(int, int) X(long, long) X(longlong, long long)            \
  X(uchar, unsigned char) X(ushort, unsigned short) X(uint, unsigned int) X(ulong, unsigned long)   \
  X(ulonglong, unsigned long long) X(int8, int8_t) X(int16, int16_t) X(int32, int32_t)              \
  X(int64, int64_t) X(uint8, uint8_t) X(uint16, uint16_t) X(uint32, uint32_t) X(uint64, uint64_t)   \
  X(size, size_t) X(ptrdiff, ptrdiff_t)

#define BSHMEM_SIZES(X) X(8, int8_t) X(16, int16_t) X(32, int32_t) X(64, int64_t) X(128, int4)

#define BSHMEM_WAIT_TYPES(X)                                                                        \
  X(short, short) X(int, int) X(long, long) X(longlong, long long) X(ushort, unsigned short)        \
  X(uint, unsigned int) X(ulong, unsigned long) X(ulonglong, unsigned long long) X(int32, int32_t)  \
  X(int64, int64_t) X(uint32, uint32_t) X(uint64, uint64_t) X(size, size_t) X(ptrdiff, ptrdiff_t)

#define BSHMEM_BITWISE_REDUCE_TYPES(X)                                                              \
  X(uchar, unsigned char) X(ushort, unsigned short) X(uint, unsigned int) X(ulong, unsigned long)   \
  X(ulonglong, unsigned long long) X(int8, int8_t) X(int16, int16_t) X(int32, int32_t)              \
  X(int64, int64_t) X(uint8, uint8_t) X(uint16, uint16_t) X(uint32, uint32_t) X(uint64, uint64_t)   \
  X(size, size_t)

#define BSHMEM_FLOAT_REDUCE_TYPES(X) X(bfloat16, __nv_bfloat16) X(half, half) X(float, float) X(double, double)

#define BSHMEM_STANDARD_REDUCE_TYPES(X)                                                             \
  BSHMEM_BITWISE_REDUCE_TYPES(X) X(char, char) X(schar, signed char) X(short, short) X(int, int)    \
  X(long, long) X(longlong, long long) BSHMEM_FLOAT_REDUCE_TYPES(X)

/* atomics */
#define BSHMEM_BITWISE_AMO_TYPES(X)                                                                 \
  X(uint, unsigned int) X(ulong, unsigned long) X(ulonglong, unsigned long long) X(int32, int32_t)  \
  X(uint32, uint32_t) X(int64, int64_t) X(uint64, uint64_t)
#define BSHMEM_STANDARD_AMO_TYPES(X)                                                                \
  BSHMEM_BITWISE_AMO_TYPES(X) X(int, int) X(long, long) X(longlong, long long) X(size, size_t) X(ptrdiff, ptrdiff_t)
#define BSHMEM_EXTENDED_AMO_TYPES(X) BSHMEM_STANDARD_AMO_TYPES(X) X(float, float) X(double, double)
// clang-format on

#ifdef __cplusplus
namespace bshmem {
// Canonical element kinds the collective kernels are instantiated for; the many
// API type names collapse onto these by size, signedness and format.
enum DType { DT_I8 = 0, DT_U8, DT_I16, DT_U16, DT_I32, DT_U32, DT_I64, DT_U64, DT_F16, DT_BF16, DT_F32, DT_F64, DT_COUNT };
template <class T> struct DTypeOf;
#define BSHMEM_DT(ctype, dt) template <> struct DTypeOf<ctype> { static constexpr int value = dt; };
BSHMEM_DT(signed char, DT_I8) BSHMEM_DT(char, DT_I8) BSHMEM_DT(unsigned char, DT_U8)
BSHMEM_DT(short, DT_I16) BSHMEM_DT(unsigned short, DT_U16)
BSHMEM_DT(int, DT_I32) BSHMEM_DT(unsigned int, DT_U32)
BSHMEM_DT(long, DT_I64) BSHMEM_DT(unsigned long, DT_U64)
BSHMEM_DT(long long, DT_I64) BSHMEM_DT(unsigned long long, DT_U64)
BSHMEM_DT(__half, DT_F16) BSHMEM_DT(__nv_bfloat16, DT_BF16) BSHMEM_DT(float, DT_F32) BSHMEM_DT(double, DT_F64)
#undef BSHMEM_DT
inline size_t dtype_size(int dt) {
  static const size_t s[DT_COUNT] = {1, 1, 2, 2, 4, 4, 8, 8, 2, 2, 4, 8};
  return dt >= 0 && dt < DT_COUNT ? s[dt] : 0;
}
}  // namespace bshmem
#endif
