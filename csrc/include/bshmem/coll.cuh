// Device collectives over the symmetric heap for sm_100a: sync/barrier,
// broadcast, fcollect (allgather), alltoall, allreduce and reducescatter for
// thread, warp, warpgroup and block scope, each usable by one CTA of a
// multi-CTA launch on its own element slice with its own row of barrier flags.
//
// The fabric is flat (every peer one NVSwitch hop away, full bandwidth), so no
// algorithm is a ring or a tree:
//   sync        one round: store my epoch into every member's flag row, wait for theirs
//               (dissemination with radix k only for thread/warp scope on big teams)
//   allreduce   one-shot pull (latency), two-shot = pull-reduce my chunk + push it to all
//               (bandwidth), NVLS one-shot / two-shot with multimem.ld_reduce / multimem.st
//   reducescatter  pull-reduce my block, or multimem.ld_reduce of it
//   fcollect / broadcast  push (vector stores) or multimem.st, then barrier; flag-in-data variants
//               without any barrier: 8-byte packets (LL) for the smallest fcollect / allreduce, 128-byte
//               packets (LL128: 120 bytes of data + an 8-byte flag) for fcollect, allreduce and broadcast
//               up to NVSHMEM_LL128_THRESHOLD bytes per PE
//   alltoall    push block p to PE p, then barrier
// 16-bit floating types accumulate in fp32 across PEs and round once.
// (reference behaviour: src/include/non_abi/device/coll/{barrier,reduce,reducescatter,fcollect,alltoall,broadcast}.cuh)
#pragma once
#include "device.cuh"
#include "nvls.cuh"

namespace bshmem {

enum ReduceOp { OP_AND = 0, OP_OR = 1, OP_XOR = 2, OP_MIN = 3, OP_MAX = 4, OP_SUM = 5, OP_PROD = 6 };
enum ReduceAlgo { RED_AUTO = 0, RED_ONESHOT_PULL = 1, RED_TWOSHOT = 2, RED_NVLS_ONESHOT = 3, RED_NVLS_TWOSHOT = 4, RED_LL = 5, RED_LL128 = 6, RED_RECEXCH = 7 };
enum FcollectAlgo { FC_AUTO = 0, FC_PUSH = 1, FC_LL = 2, FC_NVLS = 3, FC_LL128 = 4 };
enum RsAlgo { RS_AUTO = 0, RS_PULL = 1, RS_NVLS = 2 };
enum BcastAlgo { BC_AUTO = 0, BC_PUSH = 1, BC_LL = 2, BC_NVLS = 3, BC_PULL = 4 };

// ------------------------------------------------------------------ teams
__device__ __forceinline__ const bshmemi_team_t* team_ptr(int team) {
  if (team < 0 || team >= bshmemi_state_d.max_teams) return nullptr;
  return ((const bshmemi_team_t*)bshmemi_state_d.team_pool) + team;
}
__device__ __forceinline__ int team_world_pe(const bshmemi_team_t* t, int i) {
  return t->pe_of ? ((const int32_t*)t->pe_of)[i] : t->start + i * t->stride;
}
__device__ __forceinline__ int team_my_pe(int team) {
  const bshmemi_team_t* t = team_ptr(team);
  return t ? t->my_pe : -1;
}
__device__ __forceinline__ int team_n_pes(int team) {
  const bshmemi_team_t* t = team_ptr(team);
  return t && t->my_pe >= 0 ? t->size : -1;
}
__device__ __forceinline__ int team_translate_pe(int src_team, int src_pe, int dst_team) {
  const bshmemi_team_t* s = team_ptr(src_team);
  const bshmemi_team_t* d = team_ptr(dst_team);
  if (!s || !d || src_pe < 0 || src_pe >= s->size) return -1;
  const int world = team_world_pe(s, src_pe);
  if (!d->pe_of) {
    const int off = world - d->start;
    if (off < 0 || off % d->stride) return -1;
    const int idx = off / d->stride;
    return idx < d->size ? idx : -1;
  }
  for (int i = 0; i < d->size; ++i)
    if (((const int32_t*)d->pe_of)[i] == world) return i;
  return -1;
}

// ------------------------------------------------------------------ sync / barrier
// Polls a flag until it reaches `want`.  ACQUIRE = true polls with acquire loads, so the data published
// before the flag is visible to this thread on return; false leaves that to a fence of the caller.
template <bool ACQUIRE>
__device__ __forceinline__ int poll_ge(const uint64_t* flag, uint64_t want) {
  if ((ACQUIRE ? ld_acquire_sys(flag) : ld_relaxed_sys(flag)) >= want) return 0;
  const uint64_t start = global_timer_ns(), limit = bshmemi_state_d.wait_timeout_ns;
  uint32_t spins = 0;
  for (;;) {
    const uint64_t v = ACQUIRE ? ld_acquire_sys(flag) : ld_relaxed_sys(flag);
    if (v >= want) return 0;
    if ((++spins & 0xff) == 0 && global_timer_ns() - start > limit) {
      record_timeout(flag, want, v, BSHMEM_WHERE_BARRIER);
      return 1;
    }
  }
}

// Sync over the team.  One release fence for the whole group, relaxed flag stores to every member,
// acquire polls of the members' flags by the threads that own them, then a group barrier that hands
// what those threads acquired to the rest of the group: one fence on the critical path however many
// members there are.  On a flat NVSwitch fabric one all-to-all round is used (every
// member one hop away); thread and warp scope on teams beyond 32 members fall back to radix-k
// dissemination.  Returns 0, or 1 if a member did not arrive within the wait bound.
//
// The release fence has system scope: the observers of the flags are threads on other GPUs, and only a
// scope that contains both sides orders the data they read afterwards (peer pulls, multimem.ld_reduce) in
// the PTX memory model.  It also completes the group's earlier stores to peers, so sync and barrier
// (QUIET = true) cost the same here.  NVSHMEM_SYNC_GPU_SCOPE_RELEASE=1 selects a GPU-scope fence for sync
// instead: it orders this group's earlier stores to its own memory, which peers read through this GPU's
// L2, and skips the wait for stores in flight to other GPUs (a few hundred nanoseconds when there are
// some); that relies on how the hardware serves peer reads, not on the memory model, hence off by default.
template <int SCOPE, bool QUIET = false>
__device__ __forceinline__ int team_sync(const bshmemi_team_t* t, int slot = 0) {
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  group_sync<SCOPE>();
  if (size <= 1) return 0;
  uint64_t* epochs = (uint64_t*)t->epochs;
  const uint64_t epoch = epochs[slot] + 1;
  uint64_t* flags = (uint64_t*)t->sync_base + (size_t)slot * size;
  int err = 0;
  if (rank == 0) {  // release: the group's earlier stores (ordered before this by the group barrier)
    if (QUIET || !bshmemi_state_d.sync_gpu_release) fence_sys();
    else asm volatile("fence.acq_rel.gpu;" ::: "memory");
  }
  group_sync<SCOPE>();
  const int k = SCOPE == SCOPE_BLOCK || SCOPE == SCOPE_WARPGROUP || size <= 32 ? size : bshmemi_state_d.barrier_dissem_kval;
  if (k >= size) {
    for (int i = rank; i < size; i += G)
      if (i != me) st_relaxed_sys(translate(flags + me, team_world_pe(t, i)), epoch);
    for (int i = rank; i < size; i += G)
      if (i != me) err |= poll_ge<true>(flags + i, epoch);
  } else {
    // Radix-k dissemination: in round r talk to the PEs at distance j*k^r, j = 1..k-1.
    // Flag index r*(k-1)+(j-1) never exceeds `size` for k >= 2.
    int round = 0;
    for (int dist = 1; dist < size; dist *= k, ++round) {
      for (int j = 1 + rank; j < k; j += G) {
        if ((long)j * dist >= size) continue;
        const int to = (me + j * dist) % size;
        st_relaxed_sys(translate(flags + round * (k - 1) + (j - 1), team_world_pe(t, to)), epoch);
      }
      for (int j = 1 + rank; j < k; j += G) {
        if ((long)j * dist >= size) continue;
        err |= poll_ge<false>(flags + round * (k - 1) + (j - 1), epoch);
      }
      // A round's arrivals must be ordered before the next round's announcements.
      fence_sys();
      group_sync<SCOPE>();
    }
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[slot] = epoch;
  return err;
}
// Barrier = completion of this group's earlier puts (quiet) + sync; the sync's release fence is that quiet.
template <int SCOPE>
__device__ __forceinline__ int team_barrier(const bshmemi_team_t* t, int slot = 0) {
  return team_sync<SCOPE, true>(t, slot);
}

// ------------------------------------------------------------------ element arithmetic
template <class T> struct Acc { typedef T type; };
template <> struct Acc<__half> { typedef float type; };
template <> struct Acc<__nv_bfloat16> { typedef float type; };
template <class T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v) { return v; }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class A, int OP>
__device__ __forceinline__ A combine(A a, A b) {
  if (OP == OP_SUM) return a + b;
  if (OP == OP_PROD) return a * b;
  if (OP == OP_MIN) return b < a ? b : a;
  if (OP == OP_MAX) return b > a ? b : a;
  // Bitwise operators exist for integer types only; the dispatcher never
  // instantiates them for floating types, the casts keep the template well formed.
  if (OP == OP_AND) return (A)((unsigned long long)a & (unsigned long long)b);
  if (OP == OP_OR) return (A)((unsigned long long)a | (unsigned long long)b);
  return (A)((unsigned long long)a ^ (unsigned long long)b);
}

template <class T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

// acc[] op= the N elements packed in v
template <class T, int OP>
__device__ __forceinline__ void accumulate(typename Acc<T>::type* acc, uint4 v, bool first) {
  constexpr int N = VecOf<T>::N;
  T e[N];
  memcpy(e, &v, 16);
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = first ? to_acc<T>(e[j]) : combine<typename Acc<T>::type, OP>(acc[j], to_acc<T>(e[j]));
}
template <class T>
__device__ __forceinline__ uint4 pack(const typename Acc<T>::type* acc) {
  constexpr int N = VecOf<T>::N;
  T e[N];
#pragma unroll
  for (int j = 0; j < N; ++j) e[j] = from_acc<T>(acc[j]);
  uint4 v;
  memcpy(&v, e, 16);
  return v;
}

// Reduces elements [lo, hi) of `src` over all members by pulling from each
// member's copy, starting with the PE after me so that the members do not all
// read the same peer at once.  `src_off` shifts the source (reducescatter).
// Result goes to dst[i - lo + dst_off]; with PUSH_ALL it is stored to every
// member's dst (two-shot second phase fused into the first).
template <class T, int OP, int SCOPE, bool PUSH_ALL>
__device__ __forceinline__ void pull_reduce_range(const bshmemi_team_t* t, T* dst, const T* src, size_t lo, size_t hi) {
  typedef typename Acc<T>::type A;
  constexpr int N = VecOf<T>::N;
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const bool vec_ok = (((uintptr_t)(src + lo) | (uintptr_t)(dst + lo)) & 15) == 0;
  size_t nvec = vec_ok ? (hi - lo) / N : 0;
  for (size_t v = rank; v < nvec; v += G) {
    const size_t i = lo + v * N;
    A acc[N];
    for (int s = 0; s < size; ++s) {
      const int p = (me + 1 + s) % size;
      const uint4 x = *(const uint4*)translate(src + i, team_world_pe(t, p));
      accumulate<T, OP>(acc, x, s == 0);
    }
    const uint4 out = pack<T>(acc);
    if (PUSH_ALL) {
      for (int s = 0; s < size; ++s) *(uint4*)translate(dst + i, team_world_pe(t, (me + s) % size)) = out;
    } else {
      *(uint4*)(dst + i) = out;
    }
  }
  for (size_t i = lo + nvec * N + rank; i < hi; i += G) {  // ragged tail or unaligned buffers
    A acc = A();
    for (int s = 0; s < size; ++s) {
      const int p = (me + 1 + s) % size;
      const A x = to_acc<T>(*translate(src + i, team_world_pe(t, p)));
      acc = s == 0 ? x : combine<A, OP>(acc, x);
    }
    const T out = from_acc<T>(acc);
    if (PUSH_ALL) {
      for (int s = 0; s < size; ++s) *translate(dst + i, team_world_pe(t, (me + s) % size)) = out;
    } else {
      dst[i] = out;
    }
  }
}

// Splits [0, n) into `parts` contiguous pieces on vector boundaries.
template <class T>
__device__ __forceinline__ void split_range(size_t n, int parts, int which, size_t* lo, size_t* hi) {
  constexpr size_t N = VecOf<T>::N;
  const size_t nvec = (n + N - 1) / N;
  const size_t per = (nvec + parts - 1) / parts;
  size_t a = per * which * N, b = per * (which + 1) * N;
  *lo = a < n ? a : n;
  *hi = b < n ? b : n;
}

// ------------------------------------------------------------------ LL128: 128-byte packets, flag in the data
// A packet is one 128-byte line: 120 bytes of payload followed by an 8-byte flag that carries the generation of
// the call.  Eight consecutive lanes of a warp write (or read) one packet with ONE 16-byte access each, issued by the
// same instruction, so the line travels and lands as a unit: a reader that finds the flag of the generation it
// waits for has the 120 bytes that were written with it, and no barrier or separate signal is needed.  A warp moves
// four packets per instruction.  Messages must be 8-byte aligned multiples of 8 bytes; scopes must be made of whole
// warps (warp, warpgroup, block).  The packets of a team live in its LL128 area:
//   [ two generations x size x max_packets  : fcollect / allreduce, slot `my_pe` of every member ]
//   [ two generations x max_packets         : broadcast ]
//   [ size x 8 bytes                        : broadcast acknowledgements ]
// (reference: src/include/non_abi/device/common/nvshmemi_common_device.cuh:699-920, packLL128 / recvLL128;
//  src/include/non_abi/device/coll/fcollect.cuh:100-314; src/include/non_abi/device/coll/broadcast.cuh:151-334)
constexpr int LL128_DATA = 120, LL128_LINE = 128;
__device__ __forceinline__ size_t ll128_packets(size_t bytes) { return (bytes + LL128_DATA - 1) / LL128_DATA; }
struct Ll128Layout {
  size_t max_packets;   // per message
  char* exchange;       // [2][size][max_packets] lines
  char* bcast;          // [2][max_packets] lines
  uint64_t* acks;       // [size]
};
__device__ __forceinline__ Ll128Layout ll128_layout(const bshmemi_team_t* t) {
  Ll128Layout l;
  const size_t size = (size_t)t->size;
  // area = 2*size*P*128 + 2*P*128 + size*8 (rounded up by the host)  =>  P = (bytes - size*8) / (256*(size+1))
  l.max_packets = t->ll128_bytes > size * 8 ? (t->ll128_bytes - size * 8) / (2 * LL128_LINE * (size + 1)) : 0;
  l.exchange = (char*)t->ll128_base;
  l.bcast = l.exchange + 2 * size * l.max_packets * LL128_LINE;
  l.acks = (uint64_t*)(l.bcast + 2 * l.max_packets * LL128_LINE);
  return l;
}
// The 16 bytes that lane `j` (0..7) of a packet group contributes to packet `k` of a message: payload bytes
// [k*120 + 16j, +16) for j < 7; 8 payload bytes and the flag for j == 7.  Bytes past the end of the message are zero.
__device__ __forceinline__ uint4 ll128_piece(const char* msg, size_t bytes, size_t k, int j, uint64_t flag) {
  const size_t off = k * LL128_DATA + (size_t)j * 16;
  uint64_t lo = 0, hi = 0;
  if (off < bytes) lo = *(const uint64_t*)(msg + off);
  if (j == 7) hi = flag;
  else if (off + 8 < bytes) hi = *(const uint64_t*)(msg + off + 8);
  return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
}
__device__ __forceinline__ void ll128_store_line(char* line, int j, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(line + j * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ll128_load_line(const char* line, int j) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(line + j * 16) : "memory");
  return v;
}
// Whole-warp call: lane group g = lane/8 reads packet `line` (null for a group with nothing to read) until its flag is
// `flag`; returns this lane's 16 bytes.  `*err` is set if the bound of all device waits runs out.
__device__ __forceinline__ uint4 ll128_wait_line(const char* line, int lane, uint64_t flag, uint64_t start, int* err) {
  const int j = lane & 7, leader = (lane & ~7) + 7;
  uint4 v = make_uint4(0, 0, 0, 0);
  uint32_t spins = 0;
  for (;;) {
    if (line) v = ll128_load_line(line, j);
    const uint64_t seen = ((uint64_t)__shfl_sync(0xffffffffu, v.w, leader) << 32) | __shfl_sync(0xffffffffu, v.z, leader);
    const bool ok = !line || seen == flag;
    if (__all_sync(0xffffffffu, ok)) return v;
    if ((++spins & 0xff) == 0 && global_timer_ns() - start > bshmemi_state_d.wait_timeout_ns) {
      if (!ok && j == 7) record_timeout(line + LL128_DATA, flag, seen, BSHMEM_WHERE_COLL);
      *err = 1;
      return v;
    }
  }
}
// Writes this lane's payload bytes of packet `k` to the message at `msg` (bytes past the end are dropped).
__device__ __forceinline__ void ll128_unpack(char* msg, size_t bytes, size_t k, int j, uint4 v) {
  const size_t off = k * LL128_DATA + (size_t)j * 16;
  if (off < bytes) *(uint64_t*)(msg + off) = ((uint64_t)v.y << 32) | v.x;
  if (j != 7 && off + 8 < bytes) *(uint64_t*)(msg + off + 8) = ((uint64_t)v.w << 32) | v.z;
}
template <int SCOPE>
__device__ __forceinline__ bool ll128_scope_ok() {
  return SCOPE != SCOPE_THREAD && (group_size<SCOPE>() & 31) == 0;
}

// fcollect: every member's `bytes` land at dst + m * bytes on every member.
template <int SCOPE>
__device__ __forceinline__ int fcollect_ll128(const bshmemi_team_t* t, void* dst, const void* src, size_t bytes, int slot) {
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const int lane = rank & 31, warp = rank >> 5, nwarps = G >> 5, j = lane & 7;
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[slot] + 1;
  const Ll128Layout L = ll128_layout(t);
  const size_t npk = ll128_packets(bytes);
  char* buf = L.exchange + (gen & 1) * ((size_t)size * L.max_packets * LL128_LINE);
  // send: packet k of my message into slot `me` of every member
  for (size_t q = warp; q * 4 < npk; q += nwarps) {
    const size_t k = q * 4 + (lane >> 3);
    if (k >= npk) continue;
    const uint4 v = ll128_piece((const char*)src, bytes, k, j, gen);
    for (int sft = 0; sft < size; ++sft) {
      const int p = (me + 1 + sft) % size;
      ll128_store_line(translate(buf + ((size_t)me * L.max_packets + k) * LL128_LINE, team_world_pe(t, p)), j, v);
    }
  }
  // receive: the packets of every member, in my own buffer
  int err = 0;
  const uint64_t start = global_timer_ns();
  const size_t total = (size_t)size * npk;
  for (size_t q = warp; q * 4 < total && !err; q += nwarps) {
    const size_t i = q * 4 + (lane >> 3);
    const bool mine = i < total;
    const size_t m = mine ? i / npk : 0, k = mine ? i % npk : 0;
    const uint4 v = ll128_wait_line(mine ? buf + (m * L.max_packets + k) * LL128_LINE : nullptr, lane, gen, start, &err);
    if (mine && !err) ll128_unpack((char*)dst + m * bytes, bytes, k, j, v);
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[slot] = gen;
  return err;
}

// allreduce: every member pushes its whole vector to every member; each member reduces the `size` copies locally.
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int allreduce_ll128(const bshmemi_team_t* t, T* dst, const T* src, size_t n, int slot) {
  typedef typename Acc<T>::type A;
  constexpr int PER8 = 8 / (int)sizeof(T);  // elements per 8-byte word
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const int lane = rank & 31, warp = rank >> 5, nwarps = G >> 5, j = lane & 7;
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[slot] + 1;
  const Ll128Layout L = ll128_layout(t);
  const size_t bytes = n * sizeof(T), npk = ll128_packets(bytes);
  char* buf = L.exchange + (gen & 1) * ((size_t)size * L.max_packets * LL128_LINE);
  for (size_t q = warp; q * 4 < npk; q += nwarps) {
    const size_t k = q * 4 + (lane >> 3);
    if (k >= npk) continue;
    const uint4 v = ll128_piece((const char*)src, bytes, k, j, gen);
    for (int sft = 0; sft < size; ++sft) {
      const int p = (me + 1 + sft) % size;
      ll128_store_line(translate(buf + ((size_t)me * L.max_packets + k) * LL128_LINE, team_world_pe(t, p)), j, v);
    }
  }
  group_sync<SCOPE>();  // in place: all of src has been sent before any of dst is written
  int err = 0;
  const uint64_t start = global_timer_ns();
  for (size_t q = warp; q * 4 < npk && !err; q += nwarps) {
    const size_t k = q * 4 + (lane >> 3);
    const bool mine = k < npk;
    A acc[2 * PER8];
    for (int m = 0; m < size; ++m) {
      const uint4 v = ll128_wait_line(mine ? buf + ((size_t)m * L.max_packets + k) * LL128_LINE : nullptr, lane, gen, start, &err);
      T e[2 * PER8];
      memcpy(e, &v, 16);
#pragma unroll
      for (int x = 0; x < 2 * PER8; ++x) acc[x] = m == 0 ? to_acc<T>(e[x]) : combine<A, OP>(acc[x], to_acc<T>(e[x]));
    }
    if (mine && !err) {
      T e[2 * PER8];
#pragma unroll
      for (int x = 0; x < 2 * PER8; ++x) e[x] = from_acc<T>(acc[x]);
      uint4 v;
      memcpy(&v, e, 16);
      ll128_unpack((char*)dst, bytes, k, j, v);  // lane 7's upper half held the flag: unpack drops it
    }
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[slot] = gen;
  return err;
}

// broadcast: the root pushes its message to every member; the others poll their own buffer.  Data flows one way, so
// a root that runs ahead could overwrite a buffer half that a slow member still reads: every member therefore
// acknowledges each broadcast to all members (an 8-byte store, nobody waits for it), and a root starts generation g
// only once all members have acknowledged g - 2, which is normally long past.  Broadcasts have their own generation
// counter (the collective-epoch word of slot 1, which no flag-in-data collective uses) and their own packet area.
template <int SCOPE>
__device__ __forceinline__ int broadcast_ll128(const bshmemi_team_t* t, void* dst, const void* src, size_t bytes, int root) {
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const int lane = rank & 31, warp = rank >> 5, nwarps = G >> 5, j = lane & 7;
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS + 1;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[0] + 1;
  const Ll128Layout L = ll128_layout(t);
  const size_t npk = ll128_packets(bytes);
  char* buf = L.bcast + (gen & 1) * (L.max_packets * LL128_LINE);
  int err = 0;
  const uint64_t start = global_timer_ns();
  if (me == root) {
    if (gen > 2) {
      for (int m = rank; m < size; m += G) err |= poll_ge<false>(L.acks + m, gen - 2);
      group_sync<SCOPE>();
    }
    for (size_t q = warp; q * 4 < npk; q += nwarps) {
      const size_t k = q * 4 + (lane >> 3);
      if (k >= npk) continue;
      const uint4 v = ll128_piece((const char*)src, bytes, k, j, gen);
      for (int sft = 1; sft < size; ++sft) ll128_store_line(translate(buf + k * LL128_LINE, team_world_pe(t, (me + sft) % size)), j, v);
      if (dst != src) ll128_unpack((char*)dst, bytes, k, j, v);
    }
  } else {
    for (size_t q = warp; q * 4 < npk && !err; q += nwarps) {
      const size_t k = q * 4 + (lane >> 3);
      const bool mine = k < npk;
      const uint4 v = ll128_wait_line(mine ? buf + k * LL128_LINE : nullptr, lane, gen, start, &err);
      if (mine && !err) ll128_unpack((char*)dst, bytes, k, j, v);
    }
  }
  group_sync<SCOPE>();  // every thread of the group is done with the buffer half
  for (int m = rank; m < size; m += G) st_relaxed_sys(translate(L.acks + me, team_world_pe(t, m)), gen);
  if (rank == 0) epochs[0] = gen;
  return err;
}

// ------------------------------------------------------------------ allreduce, flag-in-data (small messages)
// Every member pushes its `n` elements as 8-byte packets (4 bytes of payload + the 4-byte generation of
// this call) into slot `my_pe` of every member's packet buffer; each member then polls the packets of all
// members and reduces them locally.  One link crossing, no barrier: arrival of a packet is its own signal.
// The buffer halves and the generation counter are the ones the flag-in-data fcollect uses, so the two may
// be mixed freely on a team.  Needs n * sizeof(T) to be a multiple of 4 and at most ll_bytes / (4 * size).
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int allreduce_ll(const bshmemi_team_t* t, T* dst, const T* src, size_t n, int slot) {
  typedef typename Acc<T>::type A;
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[slot] + 1;
  const uint32_t flag = (uint32_t)gen;
  const size_t words = n * sizeof(T) / 4;
  uint64_t* buf = (uint64_t*)(t->ll_base + (gen & 1) * (t->ll_bytes / 2));  // [size][words] packets
  const uint32_t* s32 = (const uint32_t*)src;
  for (size_t i = rank; i < words * size; i += G) {
    const int p = (int)(i / words);
    const size_t w = i % words;
    *(volatile uint64_t*)translate(buf + (size_t)me * words + w, team_world_pe(t, p)) = ((uint64_t)flag << 32) | s32[w];
  }
  group_sync<SCOPE>();  // in place: every word of src has been sent before any of dst is written
  // One unit = the packets of max(4, sizeof(T)) bytes: one 8-byte element, one 4-byte element or two 2-byte ones.
  constexpr int UW = sizeof(T) > 4 ? (int)sizeof(T) / 4 : 1;     // packets per unit
  constexpr int UE = sizeof(T) >= 4 ? 1 : 4 / (int)sizeof(T);    // elements per unit
  const size_t units = words / UW;
  int err = 0;
  const uint64_t start = global_timer_ns(), limit = bshmemi_state_d.wait_timeout_ns;
  for (size_t u = rank; u < units; u += G) {
    A acc[UE];
    for (int p = 0; p < size; ++p) {
      uint32_t raw[UW];
#pragma unroll
      for (int k = 0; k < UW; ++k) {
        const volatile uint64_t* pk = buf + (size_t)p * words + u * UW + k;
        uint64_t packet = *pk;
        uint32_t spins = 0;
        while ((uint32_t)(packet >> 32) != flag) {
          packet = *pk;
          if ((++spins & 0xff) == 0 && global_timer_ns() - start > limit) {
            record_timeout((const void*)pk, flag, packet >> 32, BSHMEM_WHERE_COLL);
            err = 1;
            break;
          }
        }
        raw[k] = (uint32_t)packet;
      }
      T e[UE];
      memcpy(e, raw, UW * 4);
#pragma unroll
      for (int k = 0; k < UE; ++k) acc[k] = p == 0 ? to_acc<T>(e[k]) : combine<A, OP>(acc[k], to_acc<T>(e[k]));
    }
#pragma unroll
    for (int k = 0; k < UE; ++k) dst[u * UE + k] = from_acc<T>(acc[k]);
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[slot] = gen;
  return err;
}

// ------------------------------------------------------------------ allreduce by recursive exchange
// log2(size) rounds; in round r member m exchanges its running result with member m ^ (1 << r): it pushes the result
// into the partner's scratch area of that round, raises the partner's round flag and, once its own flag is up,
// combines what the partner pushed.  Teams whose size is not a power of two fold first: the members beyond the largest
// power of two hand their vector to a partner below it and get the final result back.  Every member talks to
// log2(size) peers instead of size - 1, which is what matters on fabrics where reaching a peer is expensive; on a flat
// NVSwitch it is never the automatic choice (NVSHMEM_REDUCE_ALGO=7 or an explicit algorithm argument selects it).
// The neighbour of a round is computed from the member index, so teams carry no neighbour lists.  Scratch: the team's
// reduction scratch, two halves by generation, each [max-location slots][64 round flags][rounds + 1 vectors]; the generation lives in the
// collective-epoch word of slot 2 (no flag-in-data collective uses it).
// (reference: src/include/non_abi/device/coll/reduce.cuh:1050-1156, src/host/team/team_internal.cpp:284-455)
constexpr size_t RECEXCH_OFFSET = 16 * BSHMEM_MAX_PES;
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int allreduce_recexch(const bshmemi_team_t* t, T* dst, const T* src, size_t n) {
  typedef typename Acc<T>::type A;
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS + 2;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[0] + 1;
  char* half = (char*)t->scratch_base + (gen & 1) * t->scratch_bytes;
  // The first RECEXCH_OFFSET bytes of a half belong to the max-location reduction (one pair per member).
  uint64_t* flags = (uint64_t*)(half + RECEXCH_OFFSET);                 // [64]
  T* slots = (T*)(half + RECEXCH_OFFSET + 64 * sizeof(uint64_t));       // [rounds + 1][n]
  int p2 = 1, rounds = 0;
  while (p2 * 2 <= size) { p2 *= 2; ++rounds; }
  const int extra = size - p2;                       // members p2 .. size-1 fold into 0 .. extra-1
  int err = 0;
  auto push = [&](int to, int slot_idx, const T* v) {
    T* remote = translate(slots + (size_t)slot_idx * n, team_world_pe(t, to));
    for (size_t i = rank; i < n; i += G) remote[i] = v[i];
    group_sync<SCOPE>();
    if (rank == 0) {
      fence_sys();
      st_relaxed_sys(translate(flags + slot_idx, team_world_pe(t, to)), gen);
    }
  };
  auto wait = [&](int slot_idx) {
    if (rank == 0) err |= poll_ge<true>(flags + slot_idx, gen);
    group_sync<SCOPE>();
  };
  if (dst != src) {
    for (size_t i = rank; i < n; i += G) dst[i] = src[i];
    group_sync<SCOPE>();
  }
  if (me >= p2) {
    push(me - p2, rounds, dst);      // fold in ...
    wait(rounds);                    // ... and wait for the result
    for (size_t i = rank; i < n; i += G) dst[i] = slots[(size_t)rounds * n + i];
  } else {
    if (me < extra) {
      wait(rounds);
      for (size_t i = rank; i < n; i += G) dst[i] = from_acc<T>(combine<A, OP>(to_acc<T>(dst[i]), to_acc<T>(slots[(size_t)rounds * n + i])));
      group_sync<SCOPE>();
    }
    for (int r = 0; r < rounds; ++r) {
      const int partner = me ^ (1 << r);
      push(partner, r, dst);
      wait(r);
      // Both partners combine in the same order (lower member's value first), so every member ends with the same bits.
      for (size_t i = rank; i < n; i += G) {
        const A mine = to_acc<T>(dst[i]), theirs = to_acc<T>(slots[(size_t)r * n + i]);
        dst[i] = from_acc<T>(me < partner ? combine<A, OP>(mine, theirs) : combine<A, OP>(theirs, mine));
      }
      group_sync<SCOPE>();
    }
    if (me < extra) push(me + p2, rounds, dst);
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[0] = gen;
  return err;
}

// ------------------------------------------------------------------ reduction inside the switch
// dst[0, bytes) = reduction over the team of the `bytes` at multicast address mc_src, by the calling group.
// MC_STORE: dst is a multicast address too and the result is stored to every member (second half of a
// two-shot).  Four reductions are in flight per thread.  `bytes` is a multiple of NvlsReduce<T, OP>::grain.
template <class T, int OP, int SCOPE, bool MC_STORE>
__device__ __forceinline__ void nvls_reduce_bytes(const char* mc_src, char* dst, size_t bytes) {
  const int rank = group_rank<SCOPE>();
  const size_t G = group_size<SCOPE>();
  if (NvlsReduce<T, OP>::vector16) {
    const size_t nvec = bytes / 16;
    size_t v = rank;
    for (; v + 3 * G < nvec; v += 4 * G) {
      const uint4 r0 = MultimemSum<T>::ld(mc_src + v * 16), r1 = MultimemSum<T>::ld(mc_src + (v + G) * 16);
      const uint4 r2 = MultimemSum<T>::ld(mc_src + (v + 2 * G) * 16), r3 = MultimemSum<T>::ld(mc_src + (v + 3 * G) * 16);
      if (MC_STORE) {
        multimem_st_v4(dst + v * 16, r0);
        multimem_st_v4(dst + (v + G) * 16, r1);
        multimem_st_v4(dst + (v + 2 * G) * 16, r2);
        multimem_st_v4(dst + (v + 3 * G) * 16, r3);
      } else {
        ((uint4*)dst)[v] = r0;
        ((uint4*)dst)[v + G] = r1;
        ((uint4*)dst)[v + 2 * G] = r2;
        ((uint4*)dst)[v + 3 * G] = r3;
      }
    }
    for (; v < nvec; v += G) {
      const uint4 r = MultimemSum<T>::ld(mc_src + v * 16);
      if (MC_STORE) multimem_st_v4(dst + v * 16, r);
      else ((uint4*)dst)[v] = r;
    }
  } else {
    const size_t n = bytes / sizeof(T);
    const T* s = (const T*)mc_src;
    T* d = (T*)dst;
    auto put = [&](size_t i, T r) {
      if (!MC_STORE) d[i] = r;
      else if (sizeof(T) == 8) multimem_st_u64(d + i, (uint64_t)r);
      else multimem_st_u32(d + i, (uint32_t)r);
    };
    size_t i = rank;
    for (; i + 3 * G < n; i += 4 * G) {
      const T r0 = MultimemInt<T, OP>::ld(s + i), r1 = MultimemInt<T, OP>::ld(s + i + G);
      const T r2 = MultimemInt<T, OP>::ld(s + i + 2 * G), r3 = MultimemInt<T, OP>::ld(s + i + 3 * G);
      put(i, r0);
      put(i + G, r1);
      put(i + 2 * G, r2);
      put(i + 3 * G, r3);
    }
    for (; i < n; i += G) put(i, MultimemInt<T, OP>::ld(s + i));
  }
}

// ------------------------------------------------------------------ allreduce
// `src` and `dst` are symmetric; in-place is allowed (it then uses two-shot).
// Works on elements [lo, hi) so that CTA c of a multi-CTA launch can own a slice
// (with slot = c).  Returns non-zero if a sync timed out.
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int allreduce_range(const bshmemi_team_t* t, T* dst, const T* src, size_t lo, size_t hi, int slot, int algo) {
  const int size = t->size, me = t->my_pe;
  if (size == 1) {
    if (dst != src) memcpy_group<SCOPE>(dst + lo, src + lo, (hi - lo) * sizeof(T));
    group_sync<SCOPE>();
    return 0;
  }
  const size_t bytes = (hi - lo) * sizeof(T);
  constexpr int grain = NvlsReduce<T, OP>::grain;
  const bool nvls_ok = NvlsReduce<T, OP>::supported && t->has_nvls && (bytes % grain) == 0 &&
                       (((uintptr_t)(src + lo) | (uintptr_t)(dst + lo)) & (grain - 1)) == 0;
  if (algo == RED_AUTO) algo = bshmemi_state_d.reduce_algo;
  // Flag-in-data: whole small messages only (one group owns the team's packet buffer).
  const bool ll_ok = lo == 0 && slot == 0 && bytes > 0 && (bytes & 3) == 0 && ((uintptr_t)src & 3) == 0 && 4 * bytes * size <= t->ll_bytes;
  if (algo == RED_AUTO && ll_ok && bytes <= bshmemi_state_d.fcollect_ll_threshold) algo = RED_LL;
  const bool ll128_ok = lo == 0 && slot == 0 && bytes > 0 && (bytes & 7) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 7) == 0 && ll128_scope_ok<SCOPE>() &&
                        ll128_packets(bytes) <= ll128_layout(t).max_packets;
  if (algo == RED_AUTO && ll128_ok && bytes <= bshmemi_state_d.ll128_threshold) algo = RED_LL128;
  if (algo == RED_LL) {
    if (ll_ok) return allreduce_ll<T, OP, SCOPE>(t, dst, src, hi, slot);
    algo = RED_AUTO;
  }
  if (algo == RED_LL128) {
    if (ll128_ok) return allreduce_ll128<T, OP, SCOPE>(t, dst, src, hi, slot);
    algo = RED_AUTO;
  }
  if (algo == RED_RECEXCH) {
    int rounds = 0;
    for (int p = 1; p * 2 <= size; p *= 2) ++rounds;
    const bool fits = lo == 0 && slot == 0 && RECEXCH_OFFSET + 64 * sizeof(uint64_t) + (size_t)(rounds + 1) * bytes <= t->scratch_bytes;
    if (fits) return allreduce_recexch<T, OP, SCOPE>(t, dst, src, hi);
    algo = RED_AUTO;
  }
  if (algo == RED_AUTO) {
    if (nvls_ok) algo = ((hi - lo) <= bshmemi_state_d.reduce_nvls_threshold && dst != src) ? RED_NVLS_ONESHOT : RED_NVLS_TWOSHOT;
    else algo = (bytes <= bshmemi_state_d.reduce_oneshot_threshold && dst != src) ? RED_ONESHOT_PULL : RED_TWOSHOT;
  }
  if ((algo == RED_NVLS_ONESHOT || algo == RED_NVLS_TWOSHOT) && !nvls_ok) algo = RED_TWOSHOT;
  if ((algo == RED_ONESHOT_PULL || algo == RED_NVLS_ONESHOT) && dst == src) algo = algo == RED_NVLS_ONESHOT ? RED_NVLS_TWOSHOT : RED_TWOSHOT;

  int err = team_sync<SCOPE>(t, slot);  // every member's source is ready
  if (algo == RED_ONESHOT_PULL) {
    pull_reduce_range<T, OP, SCOPE, false>(t, dst, src, lo, hi);
    err |= team_sync<SCOPE>(t, slot);  // sources may be overwritten again
  } else if (algo == RED_TWOSHOT) {
    size_t a, b;
    split_range<T>(hi - lo, size, me, &a, &b);
    pull_reduce_range<T, OP, SCOPE, true>(t, dst, src, lo + a, lo + b);
    err |= team_barrier<SCOPE>(t, slot);  // my pushes have landed, theirs too
  } else if (algo == RED_NVLS_ONESHOT) {
    const char* mc_src = (const char*)t->mc_base + ((uint64_t)(src + lo) - bshmemi_state_d.heap_base);
    nvls_reduce_bytes<T, OP, SCOPE, false>(mc_src, (char*)(dst + lo), bytes);
    err |= team_sync<SCOPE>(t, slot);
  } else {  // NVLS two-shot: reduce my chunk in the switch, multicast the result
    size_t a, b;
    split_range<T>(hi - lo, size, me, &a, &b);
    const char* mc_src = (const char*)t->mc_base + ((uint64_t)(src + lo + a) - bshmemi_state_d.heap_base);
    char* mc_dst = (char*)t->mc_base + ((uint64_t)(dst + lo + a) - bshmemi_state_d.heap_base);
    nvls_reduce_bytes<T, OP, SCOPE, true>(mc_src, mc_dst, (b - a) * sizeof(T));
    err |= team_barrier<SCOPE>(t, slot);
  }
  return err;
}
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int allreduce(int team, T* dst, const T* src, size_t n) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  return allreduce_range<T, OP, SCOPE>(t, dst, src, 0, n, 0, RED_AUTO);
}

// ------------------------------------------------------------------ reducescatter
// src holds size*nreduce elements, dst nreduce: dst = sum over members of their block `my_pe`.
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int reducescatter_range(const bshmemi_team_t* t, T* dst, const T* src, size_t nreduce, size_t lo, size_t hi, int slot, int algo) {
  const int size = t->size, me = t->my_pe;
  const T* my_block = src + (size_t)me * nreduce;
  if (size == 1) {
    memcpy_group<SCOPE>(dst + lo, my_block + lo, (hi - lo) * sizeof(T));
    group_sync<SCOPE>();
    return 0;
  }
  const size_t bytes = (hi - lo) * sizeof(T);
  constexpr int grain = NvlsReduce<T, OP>::grain;
  const bool nvls_ok = NvlsReduce<T, OP>::supported && t->has_nvls && (bytes % grain) == 0 &&
                       (((uintptr_t)(my_block + lo) | (uintptr_t)(dst + lo)) & (grain - 1)) == 0;
  if (algo == RS_AUTO) algo = bshmemi_state_d.reducescatter_algo;
  if (algo == RS_AUTO) algo = nvls_ok ? RS_NVLS : RS_PULL;
  if (algo == RS_NVLS && !nvls_ok) algo = RS_PULL;
  int err = team_sync<SCOPE>(t, slot);
  if (algo == RS_NVLS) {
    const char* mc_src = (const char*)t->mc_base + ((uint64_t)(my_block + lo) - bshmemi_state_d.heap_base);
    nvls_reduce_bytes<T, OP, SCOPE, false>(mc_src, (char*)(dst + lo), bytes);
  } else {
    // dst is indexed from 0 while the source block starts at me*nreduce: shift dst.
    pull_reduce_range<T, OP, SCOPE, false>(t, dst - (size_t)me * nreduce, src, (size_t)me * nreduce + lo, (size_t)me * nreduce + hi);
  }
  err |= team_sync<SCOPE>(t, slot);
  return err;
}
template <class T, int OP, int SCOPE>
__device__ __forceinline__ int reducescatter(int team, T* dst, const T* src, size_t nreduce) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  return reducescatter_range<T, OP, SCOPE>(t, dst, src, nreduce, 0, nreduce, 0, RS_AUTO);
}

// ------------------------------------------------------------------ fcollect (allgather)
// Flag-in-data packets: each 8-byte unit carries 4 bytes of payload and the
// 4-byte generation number of this call, so arrival of the data is its own
// signal and no barrier is needed.  Two generations of buffer alternate.
template <int SCOPE>
__device__ __forceinline__ int fcollect_ll(const bshmemi_team_t* t, void* dst, const void* src, size_t bytes, int slot) {
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS;  // collective generations live after the barrier epochs
  group_sync<SCOPE>();
  const uint64_t gen = epochs[slot] + 1;
  const uint32_t flag = (uint32_t)gen;
  const size_t words = bytes / 4;
  const size_t half = t->ll_bytes / 2;
  uint64_t* buf = (uint64_t*)(t->ll_base + (gen & 1) * half);  // [size][words] packets
  const uint32_t* s32 = (const uint32_t*)src;
  for (size_t i = rank; i < words * size; i += G) {
    const int p = (int)(i / words);
    const size_t w = i % words;
    const uint64_t packet = ((uint64_t)flag << 32) | s32[w];
    *(volatile uint64_t*)translate(buf + (size_t)me * words + w, team_world_pe(t, p)) = packet;
  }
  int err = 0;
  uint32_t* d32 = (uint32_t*)dst;
  const uint64_t start = global_timer_ns(), limit = bshmemi_state_d.wait_timeout_ns;
  for (size_t i = rank; i < words * size; i += G) {
    const volatile uint64_t* slot_ptr = buf + i;
    uint64_t packet = *slot_ptr;
    uint32_t spins = 0;
    while ((uint32_t)(packet >> 32) != flag) {
      packet = *slot_ptr;
      if ((++spins & 0xff) == 0 && global_timer_ns() - start > limit) {
        record_timeout((const void*)slot_ptr, flag, packet >> 32, BSHMEM_WHERE_COLL);
        err = 1;
        break;
      }
    }
    d32[i] = (uint32_t)packet;
  }
  group_sync<SCOPE>();
  if (rank == 0) epochs[slot] = gen;
  return err;
}

template <int SCOPE>
__device__ __forceinline__ int fcollect_bytes(const bshmemi_team_t* t, void* dst, const void* src, size_t block_bytes, size_t lo, size_t hi, int slot, int algo) {
  // Member m's block lands at dst + m*block_bytes; this call moves bytes [lo, hi) of every block.
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const size_t bytes = hi - lo;
  if (size == 1) {
    if (dst != src) memcpy_group<SCOPE>((char*)dst + lo, (const char*)src + lo, bytes);
    group_sync<SCOPE>();
    return 0;
  }
  const bool aligned16 = ((((uintptr_t)dst + (size_t)me * block_bytes + lo) | ((uintptr_t)src + lo) | bytes) & 15) == 0;
  if (algo == FC_AUTO) algo = bshmemi_state_d.fcollect_algo;
  const bool ll_ok = lo == 0 && hi == block_bytes && (bytes & 3) == 0 && ((uintptr_t)src & 3) == 0 && ((uintptr_t)dst & 3) == 0 &&
                     2 * bytes * size <= t->ll_bytes / 2;
  const bool nvls_ok = t->has_nvls && aligned16;
  const bool ll128_ok = lo == 0 && hi == block_bytes && slot == 0 && bytes > 0 && (bytes & 7) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 7) == 0 && ll128_scope_ok<SCOPE>() &&
                        ll128_packets(bytes) <= ll128_layout(t).max_packets;
  if (algo == FC_LL128 && !ll128_ok) algo = FC_AUTO;
  if (algo == FC_AUTO) {
    if (ll_ok && bytes <= bshmemi_state_d.fcollect_ll_threshold) algo = FC_LL;
    else if (ll128_ok && bytes <= bshmemi_state_d.ll128_threshold) algo = FC_LL128;
    else if (nvls_ok && bytes * size <= bshmemi_state_d.fcollect_nvls_threshold) algo = FC_NVLS;
    else algo = FC_PUSH;
  }
  if (algo == FC_LL && !ll_ok) algo = FC_PUSH;
  if (algo == FC_NVLS && !nvls_ok) algo = FC_PUSH;
  if (algo == FC_LL) return fcollect_ll<SCOPE>(t, dst, src, bytes, slot);
  if (algo == FC_LL128) return fcollect_ll128<SCOPE>(t, dst, src, bytes, slot);
  char* my_slot = (char*)dst + (size_t)me * block_bytes + lo;
  if (algo == FC_NVLS) {
    char* mc = (char*)t->mc_base + ((uint64_t)my_slot - bshmemi_state_d.heap_base);
    const uint4* s = (const uint4*)((const char*)src + lo);
    for (size_t v = rank; v < bytes / 16; v += G) multimem_st_v4(mc + v * 16, s[v]);
  } else {
    for (int sft = 0; sft < size; ++sft) {
      const int p = (me + 1 + sft) % size;  // my own copy last
      memcpy_group<SCOPE>(translate(my_slot, team_world_pe(t, p)), (const char*)src + lo, bytes);
    }
  }
  return team_barrier<SCOPE>(t, slot);
}
template <class T, int SCOPE>
__device__ __forceinline__ int fcollect(int team, T* dst, const T* src, size_t nelems) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  return fcollect_bytes<SCOPE>(t, dst, src, nelems * sizeof(T), 0, nelems * sizeof(T), 0, FC_AUTO);
}

// ------------------------------------------------------------------ alltoall
template <int SCOPE>
__device__ __forceinline__ int alltoall_bytes(const bshmemi_team_t* t, void* dst, const void* src, size_t block_bytes, size_t lo, size_t hi, int slot) {
  const int size = t->size, me = t->my_pe;
  for (int sft = 0; sft < size; ++sft) {
    const int p = (me + 1 + sft) % size;
    char* remote = translate((char*)dst + (size_t)me * block_bytes + lo, team_world_pe(t, p));
    memcpy_group<SCOPE>(remote, (const char*)src + (size_t)p * block_bytes + lo, hi - lo);
  }
  return team_barrier<SCOPE>(t, slot);
}
template <class T, int SCOPE>
__device__ __forceinline__ int alltoall(int team, T* dst, const T* src, size_t nelems) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  return alltoall_bytes<SCOPE>(t, dst, src, nelems * sizeof(T), 0, nelems * sizeof(T), 0);
}

// ------------------------------------------------------------------ broadcast
template <int SCOPE>
__device__ __forceinline__ int broadcast_bytes(const bshmemi_team_t* t, void* dst, const void* src, size_t lo, size_t hi, int root, int slot, int algo) {
  const int size = t->size, me = t->my_pe;
  const int rank = group_rank<SCOPE>(), G = group_size<SCOPE>();
  const size_t bytes = hi - lo;
  if (algo == BC_AUTO) algo = bshmemi_state_d.bcast_algo;
  const bool nvls_ok = t->has_nvls && ((((uintptr_t)dst + lo) | ((uintptr_t)src + lo) | bytes) & 15) == 0;
  // Flag-in-data (128-byte packets): whole messages of one group only, no barrier at all.
  const bool ll128_ok = lo == 0 && slot == 0 && size > 1 && bytes > 0 && (bytes & 7) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 7) == 0 && ll128_scope_ok<SCOPE>() &&
                        ll128_packets(bytes) <= ll128_layout(t).max_packets;
  if (ll128_ok && (algo == BC_LL || (algo == BC_AUTO && bytes <= bshmemi_state_d.ll128_threshold))) return broadcast_ll128<SCOPE>(t, dst, src, bytes, root);
  if (algo == BC_AUTO || algo == BC_LL) algo = nvls_ok ? BC_NVLS : BC_PUSH;
  if (algo == BC_NVLS && !nvls_ok) algo = BC_PUSH;
  if (algo == BC_PULL) {
    int err = team_sync<SCOPE>(t, slot);  // the root's source is ready
    if (me != root || dst != src) memcpy_group<SCOPE>((char*)dst + lo, translate((const char*)src + lo, team_world_pe(t, root)), bytes);
    return err | team_sync<SCOPE>(t, slot);
  }
  if (me == root) {
    if (algo == BC_NVLS) {
      char* mc = (char*)t->mc_base + ((uint64_t)dst + lo - bshmemi_state_d.heap_base);
      const uint4* s = (const uint4*)((const char*)src + lo);
      for (size_t v = rank; v < bytes / 16; v += G) multimem_st_v4(mc + v * 16, s[v]);
    } else {
      for (int sft = 1; sft <= size; ++sft) {
        const int p = (me + sft) % size;
        if (p == me && dst == src) continue;
        memcpy_group<SCOPE>(translate((char*)dst + lo, team_world_pe(t, p)), (const char*)src + lo, bytes);
      }
    }
  }
  return team_barrier<SCOPE>(t, slot);
}
template <class T, int SCOPE>
__device__ __forceinline__ int broadcast(int team, T* dst, const T* src, size_t nelems, int root) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  return broadcast_bytes<SCOPE>(t, dst, src, 0, nelems * sizeof(T), root, 0, BC_AUTO);
}

// ------------------------------------------------------------------ maxloc
// Block-wide reduction of (value, index) pairs: every member pushes its pair into
// slot `my_pe` of each member's scratch, a barrier orders them, each member scans.
template <int SCOPE>
__device__ __forceinline__ int maxloc_double2(int team, double2* dst, const double2* src) {
  const bshmemi_team_t* t = team_ptr(team);
  if (!t || t->my_pe < 0) { report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  const int size = t->size, me = t->my_pe;
  uint64_t* epochs = (uint64_t*)t->epochs + BSHMEM_SYNC_SLOTS;
  group_sync<SCOPE>();
  const uint64_t gen = epochs[0] + 1;
  double2* slots = (double2*)(t->scratch_base + (gen & 1) * t->scratch_bytes);
  const double2 mine = *src;
  for (int p = group_rank<SCOPE>(); p < size; p += group_size<SCOPE>()) {
    double2* r = translate(slots + me, team_world_pe(t, p));
    *(volatile double*)&r->x = mine.x;
    *(volatile double*)&r->y = mine.y;
  }
  int err = team_barrier<SCOPE>(t, 0);
  if (group_rank<SCOPE>() == 0) {
    double2 best;
    best.x = *(volatile double*)&slots[0].x;
    best.y = *(volatile double*)&slots[0].y;
    for (int p = 1; p < size; ++p) {
      double2 c;
      c.x = *(volatile double*)&slots[p].x;
      c.y = *(volatile double*)&slots[p].y;
      if (c.x > best.x || (c.x == best.x && c.y < best.y)) best = c;
    }
    *dst = best;
    epochs[0] = gen;
  }
  group_sync<SCOPE>();
  return err;
}

}  // namespace bshmem
