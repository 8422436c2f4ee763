// GPU-memory back end of the symmetric heap, on CUDA virtual memory management.
//
// Growth step (collective), for a chunk of `bytes` at offset `backed_`:
//   1. cuMemCreate a physical chunk on this GPU, cuMemMap it into the local
//      window, cuMemSetAccess read/write for this GPU;
//   2. export it as a POSIX file descriptor and hand a copy to every peer over
//      unix-domain sockets (SCM_RIGHTS);
//   3. import each peer's descriptor and map it at the same offset of that
//      peer's window; the imported handle is released at once, the mapping keeps
//      the memory alive;
//   4. with NVLS: PE 0 creates a multicast object of the chunk's size and shares
//      it the same way; every PE adds its device, binds its own chunk at offset 0
//      and maps the object at `mc_base + backed_`, so that `multimem` accesses at
//      `mc_base + off` reach offset `off` of every PE's heap.
// Memory is only returned in finalize(), which unmaps the multicast window and
// unbinds before anything is released.
#include <cuda_runtime_api.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>

#include "../util/cuda_dl.h"
#include "../util/env.h"
#include "../util/log.h"
#include "heap.h"

namespace bshmem {
namespace {

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Chunk {
  size_t offset, bytes;
  CUmemGenericAllocationHandle own = 0;
  CUmemGenericAllocationHandle mc = 0;
  bool mc_bound = false, mc_mapped = false;
  bool external = false;  // caller-owned memory: mapped here, never created here
};

// A multicast object of a team that does not span the world: one object covers the heap as it was backed
// when the team was made, every member's chunks bound at their heap offsets.
struct TeamMc {
  std::vector<int> members;
  uint32_t tag = 0;
  CUmemGenericAllocationHandle mc = 0;
  char* base = nullptr;
  size_t bytes = 0;       // size of the object and of the reservation
  size_t bound = 0;       // bytes bound so far (from offset 0)
  bool added = false, mapped = false, live = false;
};

class VmmHeap final : public SymmetricHeap {
 public:
  explicit VmmHeap(bool want_nvls) : want_nvls_(want_nvls) {}
  ~VmmHeap() override { finalize(); }
  const char* kind() const override { return "VMM"; }
  bool device_memory() const override { return true; }

  int init(bshmem_bootstrap_handle_t* boot, int device, size_t stride, size_t initial, size_t granularity) override {
    boot_ = boot;
    mype_ = boot->pg_rank;
    npes_ = boot->pg_size;
    d_ = cu();
    if (!d_) {
      ERROR_PRINT("VMM heap: the CUDA driver library is not available");
      return HEAP_ERR_DRIVER;
    }
    CU_CHECK_RET(d_->cuInit_(0), HEAP_ERR_DRIVER);
    CU_CHECK_RET(d_->cuDeviceGet_(&dev_, device), HEAP_ERR_DRIVER);
    ordinal_ = device;
    CUcontext ctx = nullptr;
    d_->cuCtxGetCurrent_(&ctx);
    if (!ctx) {
      CU_CHECK_RET(d_->cuDevicePrimaryCtxRetain_(&ctx, dev_), HEAP_ERR_DRIVER);
      CU_CHECK_RET(d_->cuCtxSetCurrent_(ctx), HEAP_ERR_DRIVER);
      retained_ctx_ = true;
    }
    int vmm = 0, fd_ok = 0, mc_ok = 0;
    d_->cuDeviceGetAttribute_(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev_);
    d_->cuDeviceGetAttribute_(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev_);
    d_->cuDeviceGetAttribute_(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev_);
    if (!vmm || !fd_ok) {
      ERROR_PRINT("VMM heap: device %d lacks virtual memory management or file-descriptor handles", device);
      return HEAP_ERR_DRIVER;
    }

    memset(&prop_, 0, sizeof(prop_));
    prop_.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop_.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop_.location.id = ordinal_;
    prop_.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    CU_CHECK_RET(d_->cuMemGetAllocationGranularity_(&g, &prop_, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), HEAP_ERR_DRIVER);
    granularity_ = round_up(std::max(granularity, g), g);

    // NVLS needs every PE on one node, multicast support everywhere and >1 PE.
    int32_t my_vote = want_nvls_ && mc_ok && npes_ > 1 && boot->npes_node == npes_ && d_->cuMulticastCreate_ ? 1 : 0;
    std::vector<int32_t> votes(npes_);
    if (boot->allgather(&my_vote, votes.data(), sizeof(int32_t), boot) != 0) return HEAP_ERR_EXCHANGE;
    nvls_ = std::all_of(votes.begin(), votes.end(), [](int32_t v) { return v == 1; });
    if (nvls_) {
      CUmulticastObjectProp mp{};
      mp.numDevices = (unsigned)npes_;
      mp.size = granularity_;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t mg = 0;
      if (d_->cuMulticastGetGranularity_(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg)
        granularity_ = round_up(granularity_, mg);
    }
    stride_ = round_up(stride, granularity_);

    CUdeviceptr va = 0;
    CU_CHECK_RET(d_->cuMemAddressReserve_(&va, stride_ * npes_, granularity_, 0, 0), HEAP_ERR_OOM);
    window_base_ = (char*)va;
    if (nvls_) {
      CUdeviceptr mva = 0;
      if (d_->cuMemAddressReserve_(&mva, stride_, granularity_, 0, 0) == CUDA_SUCCESS) mc_base_ = (char*)mva;
      else nvls_ = false;
      // A failed reservation on one PE must switch NVLS off everywhere.
      int32_t ok = nvls_ ? 1 : 0;
      if (boot->allgather(&ok, votes.data(), sizeof(int32_t), boot) != 0) return HEAP_ERR_EXCHANGE;
      bool all = std::all_of(votes.begin(), votes.end(), [](int32_t v) { return v == 1; });
      if (!all && mc_base_) {
        d_->cuMemAddressFree_((CUdeviceptr)mc_base_, stride_);
        mc_base_ = nullptr;
      }
      nvls_ = all;
    }

    uint64_t key = 0;
    if (mype_ == 0) key = ((uint64_t)getpid() << 32) ^ (uint64_t)(uintptr_t)this ^ (uint64_t)time(nullptr);
    std::vector<uint64_t> keys(npes_);
    if (boot->allgather(&key, keys.data(), sizeof(key), boot) != 0) return HEAP_ERR_EXCHANGE;
    if (npes_ > 1) {
      int st = fdx_.open(keys[0], mype_, npes_);
      if (st != HEAP_OK) return st;
      if (boot->barrier(boot) != 0) return HEAP_ERR_EXCHANGE;  // every socket is bound
    }
    INFO(SUB_MEM, "VMM heap: window %zu bytes per PE, growth granule %zu, NVLS %s", stride_, granularity_, nvls_ ? "on" : "off");
    return grow(round_up(std::max(initial, granularity_), granularity_));
  }

  int grow(size_t bytes) override {
    Chunk c{backed_, bytes};
    CUresult r = d_->cuMemCreate_(&c.own, bytes, &prop_, 0);
    if (r != CUDA_SUCCESS) {
      ERROR_PRINT("VMM heap: cuMemCreate(%zu) failed: %s", bytes, cu_error_string(r).c_str());
      return HEAP_ERR_OOM;
    }
    return map_chunk(c, true);
  }

  int attach_external(void* user_ptr, size_t bytes, void** mapped) override {
    // Every PE must come with a usable buffer before anything is mapped anywhere.
    Chunk c{backed_, bytes};
    c.external = true;
    int32_t ok = 1;
    if (!user_ptr || bytes == 0 || bytes % granularity_ || backed_ + bytes > stride_) ok = 0;
    if (ok) {
      CUdeviceptr range_base = 0;
      size_t range_size = 0;
      if (d_->cuMemGetAddressRange_(&range_base, &range_size, (CUdeviceptr)user_ptr) != CUDA_SUCCESS || range_base != (CUdeviceptr)user_ptr || range_size < bytes) ok = 0;
    }
    if (ok && d_->cuMemRetainAllocationHandle_(&c.own, user_ptr) != CUDA_SUCCESS) ok = 0;
    if (ok) {
      CUmemAllocationProp up{};
      if (d_->cuMemGetAllocationPropertiesFromHandle_(&up, c.own) != CUDA_SUCCESS || up.location.type != CU_MEM_LOCATION_TYPE_DEVICE || up.location.id != ordinal_ ||
          !(up.requestedHandleTypes & CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR)) {
        d_->cuMemRelease_(c.own);
        c.own = 0;
        ok = 0;
      }
    }
    std::vector<int32_t> votes(npes_);
    if (boot_->allgather(&ok, votes.data(), sizeof(int32_t), boot_) != 0) return HEAP_ERR_EXCHANGE;
    if (!std::all_of(votes.begin(), votes.end(), [](int32_t v) { return v == 1; })) {
      if (!ok) ERROR_PRINT("VMM heap: the buffer to register must be one cuMemCreate allocation on this device, shareable as a POSIX file descriptor, whose size is a multiple of %zu bytes", granularity_);
      if (c.own) d_->cuMemRelease_(c.own);
      return HEAP_ERR_ARGS;
    }
    int st = map_chunk(c, false);
    if (st == HEAP_OK) *mapped = base() + c.offset;
    return st;
  }

  int detach_external(void* mapped, size_t bytes) override {
    cudaDeviceSynchronize();
    for (auto& c : chunks_) {
      if (!c.external || !c.own || base() + c.offset != (char*)mapped || c.bytes != bytes) continue;
      if (nvls_) {
        // The multicast window covers the whole heap or nothing: with a hole in it, it goes.
        if (boot_->barrier(boot_) != 0) return HEAP_ERR_EXCHANGE;
        disable_nvls();
      }
      if (boot_->barrier(boot_) != 0) return HEAP_ERR_EXCHANGE;  // nobody touches the range any more
      for (int pe = 0; pe < npes_; ++pe) d_->cuMemUnmap_((CUdeviceptr)(peer_base(pe) + c.offset), c.bytes);
      d_->cuMemRelease_(c.own);
      c.own = 0;
      return boot_->barrier(boot_) == 0 ? HEAP_OK : HEAP_ERR_EXCHANGE;
    }
    return HEAP_ERR_ARGS;
  }

  // Maps chunk `c` (its handle in c.own) at offset backed_ of every PE's window and appends it to the heap.
  int map_chunk(Chunk c, bool to_allocator) {
    const int tmo = (int)options().BOOTSTRAP_TIMEOUT_MS;
    const size_t bytes = c.bytes;
    CUresult r;
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = ordinal_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUdeviceptr mine = (CUdeviceptr)(base() + backed_);
    CU_CHECK_RET(d_->cuMemMap_(mine, bytes, 0, c.own, 0), HEAP_ERR_DRIVER);
    CU_CHECK_RET(d_->cuMemSetAccess_(mine, bytes, &acc, 1), HEAP_ERR_DRIVER);

    if (npes_ > 1) {
      int fd = -1;
      CU_CHECK_RET(d_->cuMemExportToShareableHandle_(&fd, c.own, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), HEAP_ERR_DRIVER);
      std::vector<int> fds;
      int st = fdx_.allgather_fd(fd, seq_++, &fds, tmo);
      ::close(fd);
      if (st != HEAP_OK) {
        ERROR_PRINT("VMM heap: exchanging chunk handles failed");
        return st;
      }
      for (int pe = 0; pe < npes_; ++pe) {
        if (pe == mype_) continue;
        CUmemGenericAllocationHandle ph = 0;
        r = d_->cuMemImportFromShareableHandle_(&ph, (void*)(uintptr_t)fds[pe], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        ::close(fds[pe]);
        if (r != CUDA_SUCCESS) {
          ERROR_PRINT("VMM heap: importing PE %d's chunk failed: %s", pe, cu_error_string(r).c_str());
          return HEAP_ERR_DRIVER;
        }
        CUdeviceptr at = (CUdeviceptr)(peer_base(pe) + backed_);
        CU_CHECK_RET(d_->cuMemMap_(at, bytes, 0, ph, 0), HEAP_ERR_DRIVER);
        CU_CHECK_RET(d_->cuMemSetAccess_(at, bytes, &acc, 1), HEAP_ERR_DRIVER);
        d_->cuMemRelease_(ph);
      }
    }
    if (nvls_) {
      int st = bind_multicast(&c, acc, tmo);
      if (st != HEAP_OK) return st;
    }
    chunks_.push_back(c);
    if (to_allocator) alloc_.add_chunk(backed_, bytes);
    backed_ += bytes;
    ++nchunks_;
    INFO(SUB_MEM, "VMM heap grew to %zu bytes (%d chunks)", backed_, nchunks_);
    return boot_->barrier(boot_) == 0 ? HEAP_OK : HEAP_ERR_EXCHANGE;
  }

  int bind_multicast(Chunk* c, const CUmemAccessDesc& acc, int tmo) {
    CUmulticastObjectProp mp{};
    mp.numDevices = (unsigned)npes_;
    mp.size = c->bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int fd = -1;
    int32_t ok = 1;
    if (mype_ == 0) {
      CUresult r = d_->cuMulticastCreate_(&c->mc, &mp);
      if (r == CUDA_SUCCESS) r = d_->cuMemExportToShareableHandle_(&fd, c->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) {
        WARN("NVLS: creating the multicast object failed (%s); multimem paths are off", cu_error_string(r).c_str());
        ok = 0;
      }
    }
    // Everyone learns whether PE 0 has an object before anyone waits for it.
    std::vector<int32_t> votes(npes_);
    if (boot_->allgather(&ok, votes.data(), sizeof(int32_t), boot_) != 0) return HEAP_ERR_EXCHANGE;
    if (!votes[0]) {
      disable_nvls();
      return HEAP_OK;
    }
    int st = fdx_.bcast_fd(0, &fd, seq_++, tmo);
    if (st != HEAP_OK) return st;
    if (mype_ != 0) {
      CUresult r = d_->cuMemImportFromShareableHandle_(&c->mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) ok = 0;
    }
    if (fd >= 0) ::close(fd);
    if (ok && d_->cuMulticastAddDevice_(c->mc, dev_) != CUDA_SUCCESS) ok = 0;
    if (boot_->allgather(&ok, votes.data(), sizeof(int32_t), boot_) != 0) return HEAP_ERR_EXCHANGE;  // also: all devices added
    bool all = std::all_of(votes.begin(), votes.end(), [](int32_t v) { return v == 1; });
    if (all) {
      CUresult r = d_->cuMulticastBindMem_(c->mc, 0, c->own, 0, c->bytes, 0);
      if (r == CUDA_SUCCESS) {
        c->mc_bound = true;
        CUdeviceptr at = (CUdeviceptr)(mc_base_ + c->offset);
        r = d_->cuMemMap_(at, c->bytes, 0, c->mc, 0);
        if (r == CUDA_SUCCESS) {
          c->mc_mapped = true;
          r = d_->cuMemSetAccess_(at, c->bytes, &acc, 1);
        }
      }
      if (r != CUDA_SUCCESS) {
        WARN("NVLS: binding or mapping failed (%s)", cu_error_string(r).c_str());
        ok = 0;
      }
      if (boot_->allgather(&ok, votes.data(), sizeof(int32_t), boot_) != 0) return HEAP_ERR_EXCHANGE;
      all = std::all_of(votes.begin(), votes.end(), [](int32_t v) { return v == 1; });
    }
    if (!all) {  // undo on every PE: the multicast window is all-or-nothing
      drop_multicast(c);
      disable_nvls();
      WARN("NVLS disabled: not every PE could join the multicast object");
    }
    return HEAP_OK;
  }

  // Switches the multicast window off for good: earlier chunks lose their
  // binding too, so that `mc_base()` is either valid for the whole heap or null.
  void disable_nvls() {
    for (size_t i = 0; i < team_mc_.size(); ++i) team_mc_drop((int)i);
    for (auto& c : chunks_) drop_multicast(&c);
    if (mc_base_) d_->cuMemAddressFree_((CUdeviceptr)mc_base_, stride_);
    mc_base_ = nullptr;
    nvls_ = false;
  }

  void drop_multicast(Chunk* c) {
    if (c->mc_mapped) d_->cuMemUnmap_((CUdeviceptr)(mc_base_ + c->offset), c->bytes);
    if (c->mc_bound) d_->cuMulticastUnbind_(c->mc, dev_, 0, c->bytes);
    if (c->mc) d_->cuMemRelease_(c->mc);
    c->mc = 0;
    c->mc_bound = c->mc_mapped = false;
  }

  // ---- team windows
  int team_mc_create(const std::vector<int>& members, uint32_t tag, int* id) override {
    *id = -1;
    if (!nvls_ || members.size() < 2) return HEAP_ERR_ARGS;
    size_t slot = 0;
    while (slot < team_mc_.size() && team_mc_[slot].live) ++slot;
    if (slot == team_mc_.size()) team_mc_.emplace_back();
    TeamMc& t = team_mc_[slot];
    t = TeamMc{};
    t.members = members;
    t.tag = tag;
    t.bytes = backed_;
    t.live = true;
    *id = (int)slot;
    if (mype_ != members[0]) return HEAP_OK;
    CUmulticastObjectProp mp{};
    mp.numDevices = (unsigned)members.size();
    mp.size = t.bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUresult r = d_->cuMulticastCreate_(&t.mc, &mp);
    if (r != CUDA_SUCCESS) {
      WARN("NVLS: no multicast object for a team of %zu PEs (%s); the team uses the peer-to-peer algorithms", members.size(), cu_error_string(r).c_str());
      t.mc = 0;
      return HEAP_ERR_DRIVER;
    }
    return HEAP_OK;
  }

  int team_mc_join(int id, int timeout_ms) override {
    if (id < 0 || id >= (int)team_mc_.size() || !team_mc_[id].live) return HEAP_ERR_ARGS;
    TeamMc& t = team_mc_[id];
    const int root = t.members[0];
    int fd = -1;
    if (mype_ == root) {
      if (d_->cuMemExportToShareableHandle_(&fd, t.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) return HEAP_ERR_DRIVER;
    }
    // Sequence numbers of team exchanges live in their own range: only the members take part.
    int st = fdx_.bcast_fd_group(root, t.members, &fd, 0x80000000u | t.tag, timeout_ms);
    if (st != HEAP_OK) {
      if (mype_ == root && fd >= 0) ::close(fd);
      return st;
    }
    CUresult r = CUDA_SUCCESS;
    if (mype_ != root) r = d_->cuMemImportFromShareableHandle_(&t.mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    if (fd >= 0) ::close(fd);
    if (r != CUDA_SUCCESS) {
      t.mc = 0;
      return HEAP_ERR_DRIVER;
    }
    if (d_->cuMulticastAddDevice_(t.mc, dev_) != CUDA_SUCCESS) return HEAP_ERR_DRIVER;
    t.added = true;
    return HEAP_OK;
  }

  int team_mc_bind(int id, char** base, size_t* bytes) override {
    if (id < 0 || id >= (int)team_mc_.size() || !team_mc_[id].live || !team_mc_[id].added) return HEAP_ERR_ARGS;
    TeamMc& t = team_mc_[id];
    for (auto& c : chunks_) {
      if (c.offset + c.bytes > t.bytes) break;
      if (!c.own) return HEAP_ERR_ARGS;  // a detached external range left a hole: no window
      CUresult r = d_->cuMulticastBindMem_(t.mc, c.offset, c.own, 0, c.bytes, 0);
      if (r != CUDA_SUCCESS) {
        WARN("NVLS: binding a team window failed (%s)", cu_error_string(r).c_str());
        return HEAP_ERR_DRIVER;
      }
      t.bound = c.offset + c.bytes;
    }
    CUdeviceptr va = 0;
    if (d_->cuMemAddressReserve_(&va, t.bytes, granularity_, 0, 0) != CUDA_SUCCESS) return HEAP_ERR_OOM;
    t.base = (char*)va;
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = ordinal_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUresult r = d_->cuMemMap_(va, t.bytes, 0, t.mc, 0);
    if (r == CUDA_SUCCESS) {
      t.mapped = true;
      r = d_->cuMemSetAccess_(va, t.bytes, &acc, 1);
    }
    if (r != CUDA_SUCCESS) {
      WARN("NVLS: mapping a team window failed (%s)", cu_error_string(r).c_str());
      return HEAP_ERR_DRIVER;
    }
    *base = t.base;
    *bytes = t.bytes;
    INFO(SUB_TEAM, "NVLS window for a team of %zu PEs: %zu bytes at %p", t.members.size(), t.bytes, (void*)t.base);
    return HEAP_OK;
  }

  void team_mc_drop(int id) override {
    if (id < 0 || id >= (int)team_mc_.size() || !team_mc_[id].live) return;
    TeamMc& t = team_mc_[id];
    if (t.mapped) d_->cuMemUnmap_((CUdeviceptr)t.base, t.bytes);
    if (t.base) d_->cuMemAddressFree_((CUdeviceptr)t.base, t.bytes);
    if (t.bound) d_->cuMulticastUnbind_(t.mc, dev_, 0, t.bound);
    if (t.mc) d_->cuMemRelease_(t.mc);
    t = TeamMc{};
  }

  void release_multicast_local() override {
    if (!window_base_) return;
    cudaDeviceSynchronize();
    for (size_t i = 0; i < team_mc_.size(); ++i) team_mc_drop((int)i);
    for (auto& c : chunks_) drop_multicast(&c);
    if (mc_base_) d_->cuMemAddressFree_((CUdeviceptr)mc_base_, stride_);
    mc_base_ = nullptr;
    nvls_ = false;
  }

  int zero(void* p, size_t bytes) override {
    return cudaMemset(p, 0, bytes) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess ? HEAP_OK : HEAP_ERR_DRIVER;
  }

  int finalize() override {
    if (!window_base_) return HEAP_OK;
    cudaDeviceSynchronize();
    // Multicast first: no PE may release memory that is still bound.
    for (size_t i = 0; i < team_mc_.size(); ++i) team_mc_drop((int)i);
    for (auto& c : chunks_) drop_multicast(&c);
    if (boot_ && npes_ > 1) boot_->barrier(boot_);
    for (auto& c : chunks_) {
      if (!c.own) continue;  // an external range that was detached
      for (int pe = 0; pe < npes_; ++pe) d_->cuMemUnmap_((CUdeviceptr)(peer_base(pe) + c.offset), c.bytes);
      d_->cuMemRelease_(c.own);
    }
    chunks_.clear();
    d_->cuMemAddressFree_((CUdeviceptr)window_base_, stride_ * npes_);
    if (mc_base_) d_->cuMemAddressFree_((CUdeviceptr)mc_base_, stride_);
    window_base_ = mc_base_ = nullptr;
    backed_ = 0;
    fdx_.close_all();
    if (retained_ctx_) d_->cuDevicePrimaryCtxRelease_(dev_);
    retained_ctx_ = false;
    return HEAP_OK;
  }

 private:
  const CuTable* d_ = nullptr;
  CUdevice dev_ = 0;
  int ordinal_ = 0;
  bool want_nvls_ = false, nvls_ = false, retained_ctx_ = false;
  CUmemAllocationProp prop_;
  std::vector<Chunk> chunks_;
  std::vector<TeamMc> team_mc_;
  FdExchange fdx_;
  uint32_t seq_ = 1;

 public:
  bool nvls() const { return nvls_; }
};

}  // namespace

std::unique_ptr<SymmetricHeap> make_vmm_heap(bool want_nvls) { return std::unique_ptr<SymmetricHeap>(new VmmHeap(want_nvls)); }

}  // namespace bshmem
