// CPU versions of the data collectives for the host-memory heap (no GPU): every member reads the other
// members' source buffers through the process-shared mapping, between two team syncs.  Same argument
// conventions and the same accumulation rule as the device code (16-bit floating types accumulate in
// fp32), so the Python layer and the API semantics can be exercised on a machine without a GPU.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

#include <algorithm>
#include <type_traits>
#include <vector>

#include "../../include/bshmem/types.h"
#include "../state/runtime.h"
#include "../util/log.h"

namespace bshmem {

enum EmulOp { E_AND = 0, E_OR = 1, E_XOR = 2, E_MIN = 3, E_MAX = 4, E_SUM = 5, E_PROD = 6 };  // = device ReduceOp

namespace {

template <class T> struct AccOf { typedef T type; };
template <> struct AccOf<__half> { typedef float type; };
template <> struct AccOf<__nv_bfloat16> { typedef float type; };
template <class T> typename AccOf<T>::type load(const T* p) { return *p; }
template <> float load<__half>(const __half* p) { return __half2float(*p); }
template <> float load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <class T> void store(T* p, typename AccOf<T>::type v) { *p = v; }
template <> void store<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> void store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <class A>
bool combine(A* acc, A x, int op) {
  switch (op) {
    case E_SUM: *acc = *acc + x; return true;
    case E_PROD: *acc = *acc * x; return true;
    case E_MIN: *acc = x < *acc ? x : *acc; return true;
    case E_MAX: *acc = x > *acc ? x : *acc; return true;
    default: break;
  }
  if constexpr (std::is_integral<A>::value) {
    if (op == E_AND) { *acc = (A)(*acc & x); return true; }
    if (op == E_OR) { *acc = (A)(*acc | x); return true; }
    if (op == E_XOR) { *acc = (A)(*acc ^ x); return true; }
  }
  return false;  // bitwise operator on a floating type
}

// dst[i] = op over members m of src_m[src_off + i], i in [0, n): members in rank order starting after me,
// as the device's pull reduction does.
template <class T>
int reduce_typed(Runtime& r, Team* t, T* dst, const T* src, size_t src_off, size_t n, int op) {
  typedef typename AccOf<T>::type A;
  for (size_t i = 0; i < n; ++i) {
    A acc = A();
    for (int s = 0; s < t->size; ++s) {
      const int m = (t->my_pe + 1 + s) % t->size;
      const T* peer = (const T*)r.heap->translate(src + src_off + i, t->members[m]);
      if (!peer) return ST_INVALID_VALUE;
      const A x = load<T>(peer);
      if (s == 0) acc = x;
      else if (!combine<A>(&acc, x, op)) return ST_INVALID_VALUE;
    }
    store<T>(dst + i, acc);
  }
  return ST_SUCCESS;
}

int reduce_any(Runtime& r, Team* t, void* dst, const void* src, size_t src_off, size_t n, int dtype, int op) {
  switch (dtype) {
    case DT_I8: return reduce_typed(r, t, (int8_t*)dst, (const int8_t*)src, src_off, n, op);
    case DT_U8: return reduce_typed(r, t, (uint8_t*)dst, (const uint8_t*)src, src_off, n, op);
    case DT_I16: return reduce_typed(r, t, (int16_t*)dst, (const int16_t*)src, src_off, n, op);
    case DT_U16: return reduce_typed(r, t, (uint16_t*)dst, (const uint16_t*)src, src_off, n, op);
    case DT_I32: return reduce_typed(r, t, (int32_t*)dst, (const int32_t*)src, src_off, n, op);
    case DT_U32: return reduce_typed(r, t, (uint32_t*)dst, (const uint32_t*)src, src_off, n, op);
    case DT_I64: return reduce_typed(r, t, (long long*)dst, (const long long*)src, src_off, n, op);
    case DT_U64: return reduce_typed(r, t, (unsigned long long*)dst, (const unsigned long long*)src, src_off, n, op);
    case DT_F16: return reduce_typed(r, t, (__half*)dst, (const __half*)src, src_off, n, op);
    case DT_BF16: return reduce_typed(r, t, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, src_off, n, op);
    case DT_F32: return reduce_typed(r, t, (float*)dst, (const float*)src, src_off, n, op);
    case DT_F64: return reduce_typed(r, t, (double*)dst, (const double*)src, src_off, n, op);
    default: return ST_INVALID_VALUE;
  }
}

Team* member_team(int team) {
  Team* t = team_get(team);
  return t && t->my_pe >= 0 ? t : nullptr;
}

}  // namespace

int emul_reduce(int team, void* dst, const void* src, size_t n, int dtype, int op) {
  Runtime& r = rt();
  Team* t = member_team(team);
  if (!t || !r.heap->contains(src)) return ST_INVALID_VALUE;
  const size_t esize = dtype_size(dtype);
  int st = emul_team_sync(team);  // every member's source is ready
  if (st) return st;
  // In place is allowed: reduce into a private copy first, publish after everyone has read the sources.
  std::vector<char> tmp(n * esize);
  st = reduce_any(r, t, tmp.data(), src, 0, n, dtype, op);
  int st2 = emul_team_sync(team);  // sources may be overwritten again
  if (st || st2) return st ? st : st2;
  memcpy(dst, tmp.data(), n * esize);
  r.n_coll++;
  return ST_SUCCESS;
}

int emul_reducescatter(int team, void* dst, const void* src, size_t nreduce, int dtype, int op) {
  Runtime& r = rt();
  Team* t = member_team(team);
  if (!t || !r.heap->contains(src)) return ST_INVALID_VALUE;
  int st = emul_team_sync(team);
  if (st) return st;
  std::vector<char> tmp(nreduce * dtype_size(dtype));
  st = reduce_any(r, t, tmp.data(), src, (size_t)t->my_pe * nreduce, nreduce, dtype, op);
  int st2 = emul_team_sync(team);
  if (st || st2) return st ? st : st2;
  memcpy(dst, tmp.data(), tmp.size());
  r.n_coll++;
  return ST_SUCCESS;
}

// Member m's `block_bytes` land at dst + m * block_bytes on every member (push, then barrier, like the device code).
int emul_fcollect(int team, void* dst, const void* src, size_t block_bytes) {
  Runtime& r = rt();
  Team* t = member_team(team);
  if (!t || !r.heap->contains(dst)) return ST_INVALID_VALUE;
  for (int s = 1; s <= t->size; ++s) {
    const int m = (t->my_pe + s) % t->size;
    void* remote = r.heap->translate((char*)dst + (size_t)t->my_pe * block_bytes, t->members[m]);
    if (!remote) return ST_INVALID_VALUE;
    memmove(remote, src, block_bytes);
  }
  r.n_coll++;
  return emul_team_sync(team);
}

// Block m of my src goes to block my_pe of member m's dst.
int emul_alltoall(int team, void* dst, const void* src, size_t block_bytes) {
  Runtime& r = rt();
  Team* t = member_team(team);
  if (!t || !r.heap->contains(dst)) return ST_INVALID_VALUE;
  for (int s = 1; s <= t->size; ++s) {
    const int m = (t->my_pe + s) % t->size;
    void* remote = r.heap->translate((char*)dst + (size_t)t->my_pe * block_bytes, t->members[m]);
    if (!remote) return ST_INVALID_VALUE;
    memmove(remote, (const char*)src + (size_t)m * block_bytes, block_bytes);
  }
  r.n_coll++;
  return emul_team_sync(team);
}

int emul_broadcast(int team, void* dst, const void* src, size_t bytes, int root) {
  Runtime& r = rt();
  Team* t = member_team(team);
  if (!t || root < 0 || root >= t->size || !r.heap->contains(dst)) return ST_INVALID_VALUE;
  if (t->my_pe == root) {
    for (int s = 1; s <= t->size; ++s) {
      const int m = (t->my_pe + s) % t->size;
      if (m == root && dst == src) continue;
      void* remote = r.heap->translate(dst, t->members[m]);
      if (!remote) return ST_INVALID_VALUE;
      memmove(remote, src, bytes);
    }
  }
  r.n_coll++;
  return emul_team_sync(team);
}

}  // namespace bshmem
