// Symmetric heap: one virtual-address reservation holding a window per PE.
//
//   window_base ─┬─ window 0 (PE 0's memory)  ─ stride bytes
//                ├─ window 1 (PE 1's memory)
//                ├─ …
//                └─ window npes-1
//
// The local heap is window `mype`; a peer's copy of a symmetric object is at
// the same offset in that peer's window.  Windows grow in lock step: growth is
// a collective step that backs [backed, new_size) with new memory on every PE
// and maps each PE's new chunk into every other PE's view of that window.
// Two back ends:
//   * VmmHeap  – GPU memory: cuMemCreate chunks, exported as POSIX file
//                descriptors, passed over unix-domain sockets (SCM_RIGHTS),
//                imported and mapped by the peers; optionally bound to an
//                NVLink multicast object (NVLS) mapped at `mc_base`.
//   * HostHeap – POSIX shared memory, needs no GPU or driver; used when no
//                device is present and by the CPU test-suite.
// (reference behaviour: src/host/mem/mem_heap.cpp, vidmem_dynamic_vmm and
//  sysmem_static_shm heaps; src/host/team/team_internal_nvls.cpp)
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../bootstrap/bootstrap.h"
#include "allocator.h"

namespace bshmem {

enum HeapStatus { HEAP_OK = 0, HEAP_ERR_OOM = 1, HEAP_ERR_DRIVER = 2, HEAP_ERR_EXCHANGE = 3, HEAP_ERR_ARGS = 4, HEAP_ERR_ASYMMETRIC = 5 };

class SymmetricHeap {
 public:
  virtual ~SymmetricHeap() {}
  // Reserves the address range and backs the first `initial` bytes.  Collective.
  virtual int init(bshmem_bootstrap_handle_t* boot, int device, size_t stride, size_t initial, size_t granularity) = 0;
  virtual int finalize() = 0;
  virtual const char* kind() const = 0;
  virtual bool device_memory() const = 0;
  // Zero-fills local heap memory (calloc).
  virtual int zero(void* p, size_t bytes) = 0;

  // Collective allocation calls: every PE must make the same call sequence.
  void* allocate(size_t size, size_t alignment, int* status = nullptr);
  int release(void* p);
  size_t allocation_size(const void* p) const;

  int mype() const { return mype_; }
  int npes() const { return npes_; }
  char* window_base() const { return window_base_; }
  char* base() const { return window_base_ + (size_t)mype_ * stride_; }
  char* peer_base(int pe) const { return window_base_ + (size_t)pe * stride_; }
  size_t stride() const { return stride_; }
  size_t backed() const { return backed_; }
  char* mc_base() const { return mc_base_; }
  bool contains(const void* p) const { return (const char*)p >= base() && (const char*)p < base() + backed_; }
  bool contains_reserved(const void* p) const { return (const char*)p >= base() && (const char*)p < base() + stride_; }
  void* translate(const void* p, int pe) const {
    if (!contains(p) || pe < 0 || pe >= npes_) return nullptr;
    return (char*)p + ((ptrdiff_t)pe - mype_) * (ptrdiff_t)stride_;
  }
  void* mc_translate(const void* p) const {
    if (!mc_base_ || !contains(p)) return nullptr;
    return mc_base_ + ((const char*)p - base());
  }
  HeapAllocator& allocator() { return alloc_; }
  // Maps a caller-owned device allocation (made with cuMemCreate, shareable as a POSIX file descriptor,
  // a multiple of granule() bytes) into the window of every PE, at the same offset everywhere, and returns
  // this PE's symmetric address of it.  Collective; every PE passes a buffer of the same size.  The range is
  // not handed to the allocator.  (reference: nvshmemx_buffer_register_symmetric, src/host/mem/mem_heap.cpp)
  virtual int attach_external(void* user_ptr, size_t bytes, void** mapped) { (void)user_ptr; (void)bytes; (void)mapped; return HEAP_ERR_ARGS; }
  // Unmaps a range made by attach_external from every window.  Collective.  The offsets are not reused.
  virtual int detach_external(void* mapped, size_t bytes) { (void)mapped; (void)bytes; return HEAP_ERR_ARGS; }
  // ---- NVLink multicast windows for teams that do not span the world (GPU back end with NVLS only).
  // Three steps, each followed by an agreement among the callers (the team code votes between them), so that
  // no PE waits for a descriptor or binds memory after another PE has failed:
  //   team_mc_create  the team's first member creates a multicast object covering the heap as backed now;
  //   team_mc_join    the object's descriptor goes to the other members, every member adds its device;
  //   team_mc_bind    every member binds its own chunks at their heap offsets and maps the object; `*base`
  //                   is then the multicast address of heap offset 0 for this team and `*bytes` what it covers.
  // team_mc_drop undoes whatever was done (local calls only).  A window does not follow later growth of the heap.
  // (reference: src/host/team/team_internal.cpp:749-851, src/host/team/team_internal_nvls.cpp)
  virtual int team_mc_create(const std::vector<int>& members, uint32_t tag, int* id) { (void)members; (void)tag; *id = -1; return HEAP_ERR_ARGS; }
  virtual int team_mc_join(int id, int timeout_ms) { (void)id; (void)timeout_ms; return HEAP_ERR_ARGS; }
  virtual int team_mc_bind(int id, char** base, size_t* bytes) { (void)id; (void)base; (void)bytes; return HEAP_ERR_ARGS; }
  virtual void team_mc_drop(int id) { (void)id; }
  // Detaches this PE from every multicast object (unmap, unbind, release) without talking to any other PE:
  // for a process that is about to leave abnormally.  The multicast window is gone afterwards.
  virtual void release_multicast_local() {}
  size_t granule() const { return granularity_; }
  // Compares the allocator history digest across PEs (error checks).
  int check_symmetry();
  int chunks() const { return nchunks_; }

 protected:
  // Backs [backed_, backed_+bytes) on every PE and maps the peers' chunks.
  virtual int grow(size_t bytes) = 0;
  bshmem_bootstrap_handle_t* boot_ = nullptr;
  int mype_ = 0, npes_ = 1;
  char* window_base_ = nullptr;
  char* mc_base_ = nullptr;
  size_t stride_ = 0, backed_ = 0, granularity_ = 0;
  int nchunks_ = 0;
  HeapAllocator alloc_;
};

std::unique_ptr<SymmetricHeap> make_vmm_heap(bool want_nvls);
std::unique_ptr<SymmetricHeap> make_host_heap();

// ---- file-descriptor passing between the processes of one node ----
class FdExchange {
 public:
  ~FdExchange();
  // Binds this PE's abstract-namespace datagram socket; `job_key` keeps jobs apart.
  int open(uint64_t job_key, int mype, int npes);
  // Every PE contributes one descriptor and receives everyone else's
  // (`out[mype]` is left -1).  Collective; `seq` must match on all PEs.
  int allgather_fd(int my_fd, uint32_t seq, std::vector<int>* out, int timeout_ms);
  // PE `root` sends one descriptor to all the others.
  int bcast_fd(int root, int* fd_inout, uint32_t seq, int timeout_ms);
  // The same among the PEs listed in `members` only (`root` is one of them); the others do not take part.
  int bcast_fd_group(int root, const std::vector<int>& members, int* fd_inout, uint32_t seq, int timeout_ms);
  void close_all();

 private:
  int send_fd(int to_pe, int fd, uint32_t seq, int timeout_ms);
  int recv_fd(int from_pe, uint32_t seq, int* fd_out, int timeout_ms);
  struct Pending { int from; uint32_t seq; int fd; };
  std::vector<Pending> pending_;
  int sock_ = -1, mype_ = 0, npes_ = 0;
  uint64_t key_ = 0;
};

}  // namespace bshmem
