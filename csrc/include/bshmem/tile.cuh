// Tile-granular device API (namespace nvshmemx): a 2-D tile of a larger tensor,
// described by a Tensor<T, Layout<shape, stride>> whose data pointer is the
// tile's first element, is moved or reduced across PEs by one thread, warp,
// warpgroup or block.  `start_coord` is the tile's origin inside the full
// tensor and `boundary` the full extent, so tiles that hang over the edge are
// clipped element by element.  All calls are non-blocking with respect to the
// other PEs: completion is `tile_collective_wait` (a team barrier).  This is the
// interface a GEMM epilogue uses to reduce or gather its output tile by tile.
//
// The last argument of every call, `flag`, picks the row of the team's synchronisation flags that the call uses
// (flag % BSHMEM_SYNC_SLOTS).  One row serves ONE group of threads at a time: two CTAs (or warps) that run tile
// collectives on the same team at the same time must pass different values, for example blockIdx.x, the same
// value on every PE for matching calls, and again in the tile_collective_wait that completes them.  With the
// default of 0 only one group per team may be inside a tile collective at any time.
//
// Algorithms (tile_coll_algo_t):
//   NVLS_ONE_SHOT_PULL_NBI  every PE reduces the tile for itself (multimem.ld_reduce for sum of
//                           float/half/bf16 on NVLS teams, peer loads otherwise); starts with a team sync
//   NVLS_TWO_SHOT_PUSH_NBI / _PULL_NBI   `root` reduces the tile and stores the result to every PE
//   NVLS_ONE_SHOT_PUSH_NBI  gather / broadcast: the caller's tile is stored to every PE (multimem.st or peer stores)
// (reference: src/include/device/tile/nvshmemx_tile_api.hpp, src/include/device_host/nvshmem_tensor.h,
//  src/include/non_abi/device/pt-to-pt/tile.cuh)
#pragma once
#include <cuda/std/tuple>
#include <cuda/std/type_traits>
#include <limits.h>

#include "coll.cuh"

template <int v>
struct ConstInt : cuda::std::integral_constant<int, v> {
  __host__ __device__ constexpr operator int() const { return v; }
};

namespace nvshmemx {

template <class... S> using shape = cuda::std::tuple<S...>;
template <class... S> using stride = cuda::std::tuple<S...>;
template <class... Ts> __host__ __device__ constexpr shape<Ts...> make_shape(Ts const&... t) { return {t...}; }
template <class... Ts> __host__ __device__ constexpr stride<Ts...> make_stride(Ts const&... t) { return {t...}; }

template <class Shape, class Stride>
struct Layout {
  Shape shape_;
  Stride stride_;
  __host__ __device__ constexpr Layout(Shape const& s = {}, Stride const& d = {}) : shape_(s), stride_(d) {}
  __host__ __device__ constexpr Shape shape() const { return shape_; }
  __host__ __device__ constexpr Stride stride() const { return stride_; }
};
template <class Shape, class Stride>
__host__ __device__ constexpr Layout<Shape, Stride> make_layout(Shape const& s, Stride const& d) { return Layout<Shape, Stride>(s, d); }

template <typename T, class LayoutT>
struct Tensor {
  using value_type = T;
  using layout_type = LayoutT;
  T* _data;
  const LayoutT _layout;
  __host__ __device__ constexpr Tensor(T* data, LayoutT layout) : _data(data), _layout(layout) {}
  __host__ __device__ Tensor(LayoutT layout) : _data(nullptr), _layout(layout) {}
  __host__ __device__ constexpr LayoutT layout() const { return _layout; }
  __host__ __device__ T* data() { return _data; }
  __host__ __device__ constexpr auto stride() const { return _layout.stride(); }
  __host__ __device__ constexpr auto shape() const { return _layout.shape(); }
};

typedef enum { NVLS_ONE_SHOT_PUSH_NBI = 0, NVLS_ONE_SHOT_PULL_NBI = 1, NVLS_TWO_SHOT_PUSH_NBI = 2, NVLS_TWO_SHOT_PULL_NBI = 3, NVSHMEMI_TILE_COLL_ALGO_SENTINEL = INT_MAX } tile_coll_algo_t;
typedef enum { PEER_PUSH_NBI = 0, PEER_PULL_NBI = 0, REMOTE_PUSH_NBI = 1, REMOTE_PULL_NBI = 1, NVSHMEMI_TILE_ALGO_SENTINEL = INT_MAX } tile_algo_t;

namespace detail {

template <class Tuple>
__device__ __forceinline__ int dim0(const Tuple& t) { return (int)cuda::std::get<0>(t); }
template <class Tuple>
__device__ __forceinline__ int dim1(const Tuple& t) { return (int)cuda::std::get<1>(t); }

// Geometry of one tile, reduced to "rows of contiguous runs": `major` is the dimension with stride 1.
struct TileGeom {
  int rows, cols;              // extent along the strided and the contiguous dimension, after clipping
  long src_pitch, dst_pitch;   // elements between consecutive rows
  bool contiguous;             // both tensors have a unit-stride dimension, and it is the same one
};

template <class SrcT, class DstT, class Coord>
__device__ __forceinline__ TileGeom geometry(const SrcT& src, const DstT& dst, const Coord& start, const Coord& bound) {
  const int s0 = dim0(src.shape()), s1 = dim1(src.shape());
  const long ss0 = dim0(src.stride()), ss1 = dim1(src.stride());
  const long ds0 = dim0(dst.stride()), ds1 = dim1(dst.stride());
  int v0 = dim0(bound) - dim0(start), v1 = dim1(bound) - dim1(start);   // valid extent from the tile origin
  v0 = v0 < s0 ? (v0 < 0 ? 0 : v0) : s0;
  v1 = v1 < s1 ? (v1 < 0 ? 0 : v1) : s1;
  TileGeom g;
  if (ss1 == 1 && ds1 == 1) { g.rows = v0; g.cols = v1; g.src_pitch = ss0; g.dst_pitch = ds0; g.contiguous = true; }
  else if (ss0 == 1 && ds0 == 1) { g.rows = v1; g.cols = v0; g.src_pitch = ss1; g.dst_pitch = ds1; g.contiguous = true; }
  else { g.rows = v0; g.cols = v1; g.src_pitch = ss0; g.dst_pitch = ds0; g.contiguous = false; }
  return g;
}

// Visits the tile in 16-byte vectors where the run length and both addresses allow it, else element-wise.
// f_vec(src_elem_offset, dst_elem_offset) handles N elements, f_one handles one.
template <class T, int SCOPE, class FVec, class FOne>
__device__ __forceinline__ void for_each(const TileGeom& g, const T* src, const T* dst, long src_col_stride, long dst_col_stride, FVec f_vec, FOne f_one) {
  constexpr int N = 16 / sizeof(T);
  const int rank = bshmem::group_rank<SCOPE>(), G = bshmem::group_size<SCOPE>();
  const bool vec = g.contiguous && (g.cols % N) == 0 && (g.src_pitch % N) == 0 && (g.dst_pitch % N) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0;
  if (vec) {
    const int vpr = g.cols / N;
    for (long i = rank; i < (long)g.rows * vpr; i += G) {
      const long r = i / vpr, c = (i % vpr) * N;
      f_vec(r * g.src_pitch + c, r * g.dst_pitch + c);
    }
  } else {
    for (long i = rank; i < (long)g.rows * g.cols; i += G) {
      const long r = i / g.cols, c = i % g.cols;
      f_one(r * g.src_pitch + c * src_col_stride, r * g.dst_pitch + c * dst_col_stride);
    }
  }
}

template <int OP, int SCOPE, class SrcT, class DstT, class Coord>
__device__ __forceinline__ int tile_reduce_impl(int team, SrcT src, DstT dst, Coord start, Coord bound, int root, bool rooted, bool everyone, uint64_t flag) {
  typedef typename SrcT::value_type T;
  typedef typename bshmem::Acc<T>::type A;
  constexpr int N = 16 / sizeof(T);
  const bshmemi_team_t* t = bshmem::team_ptr(team);
  if (!t || t->my_pe < 0) { bshmem::report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
  const TileGeom g = geometry(src, dst, start, bound);
  const long scs = g.contiguous ? 1 : dim1(src.stride()), dcs = g.contiguous ? 1 : dim1(dst.stride());
  // Every member's source tile must be in place before anyone reads it.
  int err = bshmem::team_sync<SCOPE>(t, (int)(flag % BSHMEM_SYNC_SLOTS));
  const bool i_reduce = everyone || t->my_pe == root;
  if (!i_reduce) return err;
  const bool nvls = OP == bshmem::OP_SUM && bshmem::MultimemSum<T>::supported && t->has_nvls;
  const bool push_all = !everyone && !rooted;  // two-shot: the root's result goes to every member
  const T* s = src.data();
  T* d = dst.data();
  const int size = t->size, me = t->my_pe;
  auto store_vec = [&](long doff, uint4 v) {
    if (push_all) {
      if (t->has_nvls) bshmem::multimem_st_v4((char*)t->mc_base + ((uint64_t)(d + doff) - bshmemi_state_d.heap_base), v);
      else for (int q = 0; q < size; ++q) *(uint4*)bshmem::translate(d + doff, bshmem::team_world_pe(t, (me + q) % size)) = v;
    } else {
      *(uint4*)(d + doff) = v;
    }
  };
  auto store_one = [&](long doff, T v) {
    if (push_all) for (int q = 0; q < size; ++q) *bshmem::translate(d + doff, bshmem::team_world_pe(t, (me + q) % size)) = v;
    else d[doff] = v;
  };
  for_each<T, SCOPE>(g, s, d, scs, dcs,
      [&](long soff, long doff) {
        if (nvls) {
          store_vec(doff, bshmem::MultimemSum<T>::ld((const char*)t->mc_base + ((uint64_t)(s + soff) - bshmemi_state_d.heap_base)));
        } else {
          A acc[N];
          for (int q = 0; q < size; ++q) bshmem::accumulate<T, OP>(acc, *(const uint4*)bshmem::translate(s + soff, bshmem::team_world_pe(t, (me + 1 + q) % size)), q == 0);
          store_vec(doff, bshmem::pack<T>(acc));
        }
      },
      [&](long soff, long doff) {
        A acc = A();
        for (int q = 0; q < size; ++q) {
          const A x = bshmem::to_acc<T>(*bshmem::translate(s + soff, bshmem::team_world_pe(t, (me + 1 + q) % size)));
          acc = q == 0 ? x : bshmem::combine<A, OP>(acc, x);
        }
        store_one(doff, bshmem::from_acc<T>(acc));
      });
  return err;
}

// Stores the caller's tile to every member (push == true) or to one PE / from one PE.
template <int SCOPE, class SrcT, class DstT, class Coord>
__device__ __forceinline__ int tile_copy_impl(int team, SrcT src, DstT dst, Coord start, Coord bound, int pe, int mode /*0 put, 1 get, 2 push to all*/) {
  typedef typename SrcT::value_type T;
  const TileGeom g = geometry(src, dst, start, bound);
  const long scs = g.contiguous ? 1 : dim1(src.stride()), dcs = g.contiguous ? 1 : dim1(dst.stride());
  const T* s = src.data();
  T* d = (T*)dst.data();
  if (mode == 2) {
    const bshmemi_team_t* t = bshmem::team_ptr(team);
    if (!t || t->my_pe < 0) { bshmem::report_error(BSHMEM_ERR_BAD_TEAM); return 1; }
    const int size = t->size, me = t->my_pe;
    for_each<T, SCOPE>(g, s, d, scs, dcs,
        [&](long soff, long doff) {
          const uint4 v = *(const uint4*)(s + soff);
          if (t->has_nvls) bshmem::multimem_st_v4((char*)t->mc_base + ((uint64_t)(d + doff) - bshmemi_state_d.heap_base), v);
          else for (int q = 0; q < size; ++q) *(uint4*)bshmem::translate(d + doff, bshmem::team_world_pe(t, (me + q) % size)) = v;
        },
        [&](long soff, long doff) {
          for (int q = 0; q < size; ++q) *bshmem::translate(d + doff, bshmem::team_world_pe(t, (me + q) % size)) = s[soff];
        });
    return 0;
  }
  const T* rs = mode == 1 ? bshmem::translate(s, pe) : s;
  T* rd = mode == 0 ? bshmem::translate(d, pe) : d;
  for_each<T, SCOPE>(g, rs, rd, scs, dcs, [&](long soff, long doff) { *(uint4*)(rd + doff) = *(const uint4*)(rs + soff); }, [&](long soff, long doff) { rd[doff] = rs[soff]; });
  return 0;
}

}  // namespace detail

#define BSHMEM_TILE_SCOPE(SUF, SC)                                                                                                        \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_sum_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_SUM, SC>(team, src, dst, start, bound, root, false, algo == NVLS_ONE_SHOT_PULL_NBI || algo == NVLS_ONE_SHOT_PUSH_NBI, flag); }  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_sum_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_SUM, SC>(team, src, dst, start, bound, 0, false, true, flag); }                                  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_max_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MAX, SC>(team, src, dst, start, bound, root, false, algo == NVLS_ONE_SHOT_PULL_NBI || algo == NVLS_ONE_SHOT_PUSH_NBI, flag); }  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_max_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MAX, SC>(team, src, dst, start, bound, 0, false, true, flag); }                                  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_min_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MIN, SC>(team, src, dst, start, bound, root, false, algo == NVLS_ONE_SHOT_PULL_NBI || algo == NVLS_ONE_SHOT_PUSH_NBI, flag); }  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_min_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MIN, SC>(team, src, dst, start, bound, 0, false, true, flag); }                                  \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_sum_rooted_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_SUM, SC>(team, src, dst, start, bound, root, true, false, flag); }                               \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_max_rooted_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MAX, SC>(team, src, dst, start, bound, root, true, false, flag); }                               \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_min_rooted_reduce##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int root, uint64_t flag) { \
    return detail::tile_reduce_impl<bshmem::OP_MIN, SC>(team, src, dst, start, bound, root, true, false, flag); }                               \
  /* The caller's tile lands in `dst` (the caller's block of the gathered tensor) on every member. */                                     \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_allgather##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, uint64_t flag) { \
    return detail::tile_copy_impl<SC>(team, src, dst, start, bound, 0, 2); }                                                               \
  /* Called by the root only: its tile is stored into `dst` on every member. */                                                           \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_coll_algo_t algo>                                        \
  __device__ __forceinline__ int tile_broadcast##SUF(nvshmem_team_t team, src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, uint64_t flag) { \
    return detail::tile_copy_impl<SC>(team, src, dst, start, bound, 0, 2); }                                                               \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_algo_t algo>                                             \
  __device__ __forceinline__ int tile_put##SUF(src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int pe, uint64_t) {      \
    return detail::tile_copy_impl<SC>(0, src, dst, start, bound, pe, 0); }                                                                 \
  template <typename src_tensor_t, typename dst_tensor_t, typename tuple_t, tile_algo_t algo>                                             \
  __device__ __forceinline__ int tile_get##SUF(src_tensor_t src, dst_tensor_t dst, tuple_t start, tuple_t bound, int pe, uint64_t) {      \
    return detail::tile_copy_impl<SC>(0, src, dst, start, bound, pe, 1); }                                                                 \
  template <tile_coll_algo_t algo>                                                                                                        \
  __device__ __forceinline__ int tile_collective_wait##SUF(nvshmem_team_t team, uint64_t flag) {                                          \
    const bshmemi_team_t* t = bshmem::team_ptr(team);                                                                                     \
    return t ? bshmem::team_barrier<SC>(t, (int)(flag % BSHMEM_SYNC_SLOTS)) : 1; }

BSHMEM_TILE_SCOPE(, bshmem::SCOPE_THREAD)
BSHMEM_TILE_SCOPE(_warp, bshmem::SCOPE_WARP)
BSHMEM_TILE_SCOPE(_warpgroup, bshmem::SCOPE_WARPGROUP)
BSHMEM_TILE_SCOPE(_block, bshmem::SCOPE_BLOCK)
#undef BSHMEM_TILE_SCOPE

}  // namespace nvshmemx
