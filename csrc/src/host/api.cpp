// Definitions of the public host API.  Typed families are generated from the
// type tables; every function funnels into a few generic routines (byte copies
// to the translated peer address, stream memory operations for signals, the
// collective launchers).
// (reference behaviour: src/host/init/init.cu, src/host/mem/mem_heap.cpp:2288-2438,
//  src/host/comm/putget.cpp, sync.cpp, quiet.cpp, src/host/coll/**, src/host/team/team.cu)
#include <string.h>

#include <sched.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <type_traits>
#include <vector>

#define BSHMEM_NO_INLINE_LAUNCH  // this file defines the exported versions
#include "../../include/nvshmem_host.h"
#include "../coll/coll_host.h"
#include "../state/runtime.h"
#include "../util/cuda_dl.h"
#include "../util/env.h"
#include "../util/log.h"
#include "../util/nvtx.h"
#include "amo.h"

using namespace bshmem;

namespace {

enum CopyMode { COPY_BLOCKING, COPY_NBI, COPY_STREAM };

bool ready(const char* fn) {
  if (is_initialized()) {
    push_pending_modules();  // libraries with device code that were loaded since the last call
    return true;
  }
  ERROR_PRINT("%s called before nvshmem_init (or after finalize)", fn);
  return false;
}

cudaStream_t nbi_stream(Runtime& r, int pe) {
  int dist = (pe - r.mype + r.npes) % r.npes;
  size_t i = (size_t)dist % r.peer_streams.size();
  r.peer_stream_used[i] = true;
  return r.peer_streams[i];
}

// Copies `bytes` between a local buffer and the symmetric object on `pe`.
// put: dest symmetric; get: src symmetric.
void rma(void* dest, const void* src, size_t bytes, int pe, bool is_put, CopyMode mode, cudaStream_t stream, const char* fn) {
  if (!ready(fn) || bytes == 0) return;
  Runtime& r = rt();
  NvtxRange nvtx(mode == COPY_BLOCKING ? NVTX_RMA_BLOCKING : NVTX_RMA_NONBLOCKING, fn);
  const void* sym = is_put ? dest : src;
  void* remote = r.heap->translate(sym, pe);
  if (!remote) {
    ERROR_PRINT("%s: %p is not a symmetric address or PE %d is out of range", fn, sym, pe);
    return;
  }
  void* d = is_put ? remote : dest;
  const void* s = is_put ? src : remote;
  if (is_put) { r.n_put++; r.bytes_put += bytes; } else { r.n_get++; r.bytes_get += bytes; }
  if (!r.have_gpu) {
    memcpy(d, s, bytes);
    return;
  }
  cudaStream_t st = mode == COPY_STREAM ? stream : mode == COPY_NBI ? nbi_stream(r, pe) : r.stream;
  cudaError_t e = cudaMemcpyAsync(d, s, bytes, cudaMemcpyDefault, st);
  if (e == cudaSuccess && mode == COPY_BLOCKING) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) ERROR_PRINT("%s: copy failed: %s", fn, cudaGetErrorString(e));
}

void rma_strided(void* dest, const void* src, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, size_t esize, int pe, bool is_put, CopyMode mode,
                 cudaStream_t stream, const char* fn) {
  if (!ready(fn) || nelems == 0) return;
  Runtime& r = rt();
  const void* sym = is_put ? dest : src;
  void* remote = r.heap->translate(sym, pe);
  if (!remote) {
    ERROR_PRINT("%s: %p is not a symmetric address or PE %d is out of range", fn, sym, pe);
    return;
  }
  char* d = (char*)(is_put ? remote : dest);
  const char* s = (const char*)(is_put ? src : remote);
  if (!r.have_gpu) {
    for (size_t i = 0; i < nelems; ++i) memcpy(d + i * dst * esize, s + i * sst * esize, esize);
    return;
  }
  cudaStream_t st = mode == COPY_STREAM ? stream : r.stream;
  cudaError_t e = cudaMemcpy2DAsync(d, dst * esize, s, sst * esize, esize, nelems, cudaMemcpyDefault, st);
  if (e == cudaSuccess && mode == COPY_BLOCKING) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) ERROR_PRINT("%s: strided copy failed: %s", fn, cudaGetErrorString(e));
}

void signal_on_stream(uint64_t* sig, uint64_t value, int op, int pe, cudaStream_t stream) {
  Runtime& r = rt();
  uint64_t* remote = (uint64_t*)r.heap->translate(sig, pe);
  if (!remote) {
    ERROR_PRINT("signal: %p is not a symmetric address", (void*)sig);
    return;
  }
  r.n_signal++;
  if (!r.have_gpu) {
    if (op == NVSHMEM_SIGNAL_ADD) __atomic_fetch_add(remote, value, __ATOMIC_RELEASE);
    else __atomic_store_n(remote, value, __ATOMIC_RELEASE);
    return;
  }
  const CuTable* d = cu();
  // A stream memory operation is ordered after the copies enqueued before it and
  // costs no kernel launch; ADD needs an atomic, which only a kernel can do.
  if (op == NVSHMEM_SIGNAL_SET && r.topo.stream_memops && d && d->cuStreamWriteValue64_) {
    if (d->cuStreamWriteValue64_((CUstream)stream, (CUdeviceptr)remote, value, CU_STREAM_WRITE_VALUE_DEFAULT) == CUDA_SUCCESS) return;
  }
  p2p_signal_op_on_stream(sig, value, op, pe, stream);
}

void wait_on_stream(const void* ivar, int cmp, uint64_t value, int width, bool is_signed, cudaStream_t stream) {
  Runtime& r = rt();
  if (!r.have_gpu) {
    // Host-memory heap: the "stream" is the calling thread, which polls the word itself, with the same bound
    // as every other wait; a wait that runs out sets the time-out bit instead of blocking for ever.
    auto read = [&]() -> int64_t {
      switch (width) {
        case 8: return (int64_t)__atomic_load_n((const uint64_t*)ivar, __ATOMIC_ACQUIRE);
        case 4: return is_signed ? (int64_t)__atomic_load_n((const int32_t*)ivar, __ATOMIC_ACQUIRE) : (int64_t)__atomic_load_n((const uint32_t*)ivar, __ATOMIC_ACQUIRE);
        default: return is_signed ? (int64_t)__atomic_load_n((const int16_t*)ivar, __ATOMIC_ACQUIRE) : (int64_t)__atomic_load_n((const uint16_t*)ivar, __ATOMIC_ACQUIRE);
      }
    };
    auto holds = [&](int64_t v) {
      const bool u = width == 8 && !is_signed;  // full-width unsigned values compare as unsigned
      const uint64_t a = (uint64_t)v, b = value;
      const int64_t sb = (int64_t)value;
      switch (cmp) {
        case NVSHMEM_CMP_EQ: return a == b;
        case NVSHMEM_CMP_NE: return a != b;
        case NVSHMEM_CMP_GT: return u ? a > b : v > sb;
        case NVSHMEM_CMP_GE: return u ? a >= b : v >= sb;
        case NVSHMEM_CMP_LT: return u ? a < b : v < sb;
        case NVSHMEM_CMP_LE: return u ? a <= b : v <= sb;
        default: return true;
      }
    };
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    const long limit_ms = (long)(r.dstate.wait_timeout_ns / 1000000ull);  // follows nvshmemx_b200_set_wait_timeout_ms
    for (unsigned spins = 0; !holds(read()); ++spins) {
      if ((spins & 1023) == 1023) {
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        if ((t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000 > limit_ms) {
          if (r.status_host) status_or(&r.status_host->error_bits, BSHMEM_ERR_WAIT_TIMEOUT);
          ERROR_PRINT("wait on %p timed out after %ld ms", ivar, limit_ms);
          return;
        }
        sched_yield();
      }
    }
    return;
  }
  const CuTable* d = cu();
  if (width == 8 && !is_signed && r.topo.stream_memops && d && d->cuStreamWaitValue64_ && (cmp == NVSHMEM_CMP_GE || cmp == NVSHMEM_CMP_EQ)) {
    unsigned flags = (cmp == NVSHMEM_CMP_GE ? CU_STREAM_WAIT_VALUE_GEQ : CU_STREAM_WAIT_VALUE_EQ) | CU_STREAM_WAIT_VALUE_FLUSH;
    if (d->cuStreamWaitValue64_((CUstream)stream, (CUdeviceptr)ivar, value, flags) == CUDA_SUCCESS) return;
  }
  p2p_wait_until_on_stream(ivar, cmp, value, width, is_signed, stream);
}

int coll_finish(int st, cudaStream_t s) {  // blocking flavour of a collective launched on the internal stream
  if (st) return st;
  Runtime& r = rt();
  if (!r.have_gpu) return ST_SUCCESS;  // the CPU versions of the collectives have already run
  if (cudaStreamSynchronize(s) != cudaSuccess) return ST_INTERNAL;
  return r.status_host && (status_load(&r.status_host->error_bits) & BSHMEM_ERR_WAIT_TIMEOUT) ? ST_INTERNAL : ST_SUCCESS;
}

int do_init(unsigned int flags, nvshmemx_init_attr_t* attr, bool hostlib_only) {
  std::lock_guard<std::mutex> lk(rt().mu);
  const Options& o = options();
  std::string mode = o.BOOTSTRAP;
  std::transform(mode.begin(), mode.end(), mode.begin(), ::toupper);
  int device = -1;
  if (attr && (attr->version >> 16) >= 2) device = attr->args.cuda_device_id;
  if (flags & NVSHMEMX_INIT_WITH_SHMEM) return runtime_init(nullptr, 0, 1, device, hostlib_only, BOOT_SHMEM);  // the program has initialised OpenSHMEM
  if (flags & NVSHMEMX_INIT_WITH_MPI_COMM) {
    if (!attr || !attr->mpi_comm) return NVSHMEMX_ERROR_INVALID_VALUE;  // mpi_comm points at the caller's MPI_Comm
    return runtime_init((const bshmem_uniqueid_t*)attr->mpi_comm, 0, 1, device, hostlib_only, BOOT_MPI);
  }
  if (flags & NVSHMEMX_INIT_WITH_UNIQUEID) {
    if (!attr || !attr->args.uid_args.id) return NVSHMEMX_ERROR_INVALID_VALUE;
    return runtime_init((const bshmem_uniqueid_t*)attr->args.uid_args.id, attr->args.uid_args.myrank, attr->args.uid_args.nranks, device, hostlib_only, BOOT_UID);
  }
  if (mode == "PLUGIN") return runtime_init(nullptr, 0, 1, device, hostlib_only, BOOT_PLUGIN);
  if (mode == "MPI") return runtime_init(nullptr, 0, 1, device, hostlib_only, BOOT_MPI);
  if (mode == "SHMEM") return runtime_init(nullptr, 0, 1, device, hostlib_only, BOOT_SHMEM);
  // Started by a PMI process manager (mpiexec / nvshmrun / srun): asked for by name, or recognised by the
  // manager's variables when nothing names a rank for the unique-id bootstrap.
  if (mode == "PMI" || (bootstrap_pmi_available() && !getenv("RANK") && !getenv("NVSHMEM_BOOTSTRAP_UID_RANK")))
    return runtime_init(nullptr, 0, 1, device, hostlib_only, BOOT_PMI);
  // Plain nvshmem_init(): a launcher must have told us who we are.  torchrun-style
  // variables are understood; the session id names the root's address.
  const char* rank = getenv("NVSHMEM_BOOTSTRAP_UID_RANK") ? getenv("NVSHMEM_BOOTSTRAP_UID_RANK") : getenv("RANK");
  const char* size = getenv("NVSHMEM_BOOTSTRAP_UID_NRANKS") ? getenv("NVSHMEM_BOOTSTRAP_UID_NRANKS") : getenv("WORLD_SIZE");
  if (!rank || !size) {
    if (o.BOOTSTRAP_UID_SESSION_ID.empty()) {  // a lone process
      bshmem_uniqueid_t id;
      if (bootstrap_uid_get_unique_id(&id) != BOOT_OK) return NVSHMEMX_ERROR_INTERNAL;
      return runtime_init(&id, 0, 1, device, hostlib_only, BOOT_UID);
    }
    ERROR_PRINT("nvshmem_init: set RANK and WORLD_SIZE (or NVSHMEM_BOOTSTRAP_UID_RANK/_NRANKS) together with NVSHMEM_BOOTSTRAP_UID_SESSION_ID");
    return NVSHMEMX_ERROR_INVALID_VALUE;
  }
  if (o.BOOTSTRAP_UID_SESSION_ID.empty()) {
    ERROR_PRINT("nvshmem_init: NVSHMEM_BOOTSTRAP_UID_SESSION_ID=<addr>:<port> is needed when no unique id is passed");
    return NVSHMEMX_ERROR_INVALID_VALUE;
  }
  return runtime_init(nullptr, atoi(rank), atoi(size), device, hostlib_only, BOOT_UID);
}

}  // namespace

template <class T>
static void wait_all_impl(T* ivars, size_t n, const int* status, int cmp, const T* values, T value, cudaStream_t s) {
  // Entry by entry (on the host-memory back end the calling thread polls each word, with the usual bound).
  if (!is_initialized()) return;
  for (size_t i = 0; i < n; ++i) {
    if (status && status[i]) continue;
    wait_on_stream(ivars + i, cmp, (uint64_t)(values ? values[i] : value), (int)sizeof(T), std::is_signed<T>::value, s);
  }
}
extern "C" {

// ------------------------------------------------------------------ init / query
void nvshmem_init(void) {
  if (do_init(0, nullptr, false) != 0) ERROR_PRINT("nvshmem_init failed");
}
int nvshmem_init_thread(int, int* provided) {
  int st = do_init(0, nullptr, false);
  if (provided) *provided = NVSHMEM_THREAD_SERIALIZED;
  return st;
}
int nvshmemx_init_attr(unsigned int flags, nvshmemx_init_attr_t* attr) { return do_init(flags, attr, false); }
int nvshmemx_hostlib_init_attr(unsigned int flags, nvshmemx_init_attr_t* attr) { return do_init(flags, attr, true); }
int nvshmemx_b200_init_uid(const nvshmemx_uniqueid_t* id, int rank, int nranks, int device) {
  std::lock_guard<std::mutex> lk(rt().mu);
  return runtime_init((const bshmem_uniqueid_t*)id, rank, nranks, device, true, BOOT_UID);
}
int nvshmemx_get_uniqueid(nvshmemx_uniqueid_t* id) {
  static_assert(sizeof(nvshmemx_uniqueid_t) == sizeof(bshmem_uniqueid_t), "unique id layouts differ");
  options();
  log_init();
  return bootstrap_uid_get_unique_id((bshmem_uniqueid_t*)id) == BOOT_OK ? NVSHMEMX_SUCCESS : NVSHMEMX_ERROR_INTERNAL;
}
int nvshmemx_set_attr_uniqueid_args(int myrank, int nranks, const nvshmemx_uniqueid_t* id, nvshmemx_init_attr_t* attr) {
  if (!attr || !id) return NVSHMEMX_ERROR_INVALID_VALUE;
  attr->args.uid_args.id = (nvshmemx_uniqueid_t*)id;
  attr->args.uid_args.myrank = myrank;
  attr->args.uid_args.nranks = nranks;
  return NVSHMEMX_SUCCESS;
}
int nvshmemx_init_status(void) {
  int s = rt().init_status;
  if (s >= INIT_IS_INITIALIZED) {
    // Several PEs on one GPU are reported the way the reference reports them (reference: src/host/init/init.cu nvshmemx_init_status).
    const int mpg = rt().mpg_status;
    return mpg == MPG_FULL ? NVSHMEM_STATUS_FULL_MPG : mpg == MPG_LIMITED ? NVSHMEM_STATUS_LIMITED_MPG : NVSHMEM_STATUS_IS_INITIALIZED;
  }
  return s == INIT_IS_BOOTSTRAPPED ? NVSHMEM_STATUS_IS_BOOTSTRAPPED : NVSHMEM_STATUS_NOT_INITIALIZED;
}
void nvshmem_finalize(void) {
  std::lock_guard<std::mutex> lk(rt().mu);
  runtime_finalize();
}
void nvshmemx_hostlib_finalize(void) { nvshmem_finalize(); }
void nvshmem_global_exit(int status) {
  Runtime& r = rt();
  if (r.boot_live && r.boot.global_exit) r.boot.global_exit(status, &r.boot);
  _exit(status);
}
void nvshmem_query_thread(int* provided) {
  if (provided) *provided = NVSHMEM_THREAD_SERIALIZED;
}
int nvshmem_my_pe(void) { return rt().mype; }
int nvshmem_n_pes(void) { return rt().npes; }
void nvshmem_info_get_version(int* major, int* minor) {
  if (major) *major = NVSHMEM_MAJOR_VERSION;
  if (minor) *minor = NVSHMEM_MINOR_VERSION;
}
void nvshmem_info_get_name(char* name) {
  if (name) strncpy(name, NVSHMEM_VENDOR_STRING, NVSHMEM_MAX_NAME_LEN);
}
void nvshmemx_vendor_get_version_info(int* major, int* minor, int* patch) {
  if (major) *major = BSHMEM_MAJOR;
  if (minor) *minor = BSHMEM_MINOR;
  if (patch) *patch = BSHMEM_PATCH;
}

// A CUDA module loaded with the driver API (cuModuleLoad, cuLibraryLoad) carries its own copy of the state under
// the unmangled global name `bshmemi_state_d`, which the device headers emit when the module's source defines
// BSHMEM_DEVICE_MODULE before including them.  The copy is filled here and, like the copies of the modules that
// register themselves, again whenever the state changes (heap growth, multicast window), until the matching
// finalize call.  (reference: src/host/init/init.cu:1829-1916)
static int module_init_common(void* handle, CUdeviceptr addr, size_t bytes) {
  Runtime& r = rt();
  if (!is_initialized() || !r.have_gpu) return NVSHMEMX_ERROR_INVALID_VALUE;
  if (bytes != sizeof(bshmemi_state_t)) {
    ERROR_PRINT("the module's bshmemi_state_d has %zu bytes, this library's has %zu: it was built against other headers", bytes, sizeof(bshmemi_state_t));
    return NVSHMEMX_ERROR_SYMMETRY;
  }
  std::lock_guard<std::mutex> lk(r.mu);
  if (cudaMemcpy((void*)addr, &r.dstate, sizeof(r.dstate), cudaMemcpyHostToDevice) != cudaSuccess) return NVSHMEMX_ERROR_INTERNAL;
  for (auto& m : r.driver_modules)
    if (m.first == handle) { m.second = (void*)addr; return NVSHMEMX_SUCCESS; }
  r.driver_modules.emplace_back(handle, (void*)addr);
  return NVSHMEMX_SUCCESS;
}
static int module_finalize_common(void* handle) {
  Runtime& r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  for (size_t i = 0; i < r.driver_modules.size(); ++i)
    if (r.driver_modules[i].first == handle) {
      r.driver_modules.erase(r.driver_modules.begin() + i);
      return NVSHMEMX_SUCCESS;
    }
  return NVSHMEMX_ERROR_INVALID_VALUE;
}
int nvshmemx_cumodule_init(void* cumodule) {
  const CuTable* d = cu();
  if (!d || !d->cuModuleGetGlobal_) return NVSHMEMX_ERROR_NOT_SUPPORTED;
  CUdeviceptr addr = 0;
  size_t bytes = 0;
  if (d->cuModuleGetGlobal_(&addr, &bytes, (CUmodule)cumodule, "bshmemi_state_d") != CUDA_SUCCESS) {
    ERROR_PRINT("nvshmemx_cumodule_init: the module has no global `bshmemi_state_d` (define BSHMEM_DEVICE_MODULE before including the device headers in its source)");
    return NVSHMEMX_ERROR_INVALID_VALUE;
  }
  return module_init_common(cumodule, addr, bytes);
}
int nvshmemx_cumodule_finalize(void* cumodule) { return module_finalize_common(cumodule); }
int nvshmemx_culibrary_init(void* culibrary) {
  void* sym = nullptr;
  typedef CUresult (*get_global_t)(CUdeviceptr*, size_t*, void*, const char*);
  if (cudaGetDriverEntryPoint("cuLibraryGetGlobal", &sym, cudaEnableDefault, nullptr) != cudaSuccess || !sym) return NVSHMEMX_ERROR_NOT_SUPPORTED;
  CUdeviceptr addr = 0;
  size_t bytes = 0;
  if (((get_global_t)sym)(&addr, &bytes, culibrary, "bshmemi_state_d") != CUDA_SUCCESS) return NVSHMEMX_ERROR_INVALID_VALUE;
  return module_init_common(culibrary, addr, bytes);
}
int nvshmemx_culibrary_finalize(void* culibrary) { return module_finalize_common(culibrary); }

// ------------------------------------------------------------------ memory
static void* alloc_common(size_t size, size_t alignment, bool zero, const char* fn) {
  if (!ready(fn) || size == 0) return nullptr;
  Runtime& r = rt();
  NvtxRange nvtx(NVTX_ALLOC, fn);
  std::lock_guard<std::mutex> lk(r.mu);
  if (alignment && (alignment & (alignment - 1))) {
    ERROR_PRINT("%s: alignment %zu is not a power of two", fn, alignment);
    return nullptr;
  }
  int hst = 0;
  const size_t before = r.heap->backed();
  void* p = r.heap->allocate(size, alignment, &hst);
  if (!p) {
    ERROR_PRINT("%s(%zu) failed (status %d)", fn, size, hst);
    return nullptr;
  }
  if (r.heap->backed() != before) {  // the heap grew: republish its size
    r.dstate.heap_size = r.heap->backed();
    r.dstate.mc_base = (uint64_t)r.heap->mc_base();
    r.dstate.nvls_world = r.heap->mc_base() != nullptr;
    teams_drop_windows(r);
    push_device_state();
  }
  if (options().ENABLE_ERROR_CHECKS && r.heap->check_symmetry() != HEAP_OK) return nullptr;
  if (zero) r.heap->zero(p, size);
  r.n_alloc++;
  // Allocation is collective: nobody uses the new object before everyone has it.
  host_barrier_all_blocking();
  return p;
}
void* nvshmem_malloc(size_t size) { return alloc_common(size, 0, false, "nvshmem_malloc"); }
void* nvshmem_calloc(size_t count, size_t size) {
  if (size && count > SIZE_MAX / size) return nullptr;
  return alloc_common(count * size, 0, true, "nvshmem_calloc");
}
void* nvshmem_align(size_t alignment, size_t size) { return alloc_common(size, alignment, false, "nvshmem_align"); }
void nvshmem_free(void* ptr) {
  if (!ptr || !ready("nvshmem_free")) return;
  Runtime& r = rt();
  NvtxRange nvtx(NVTX_ALLOC, "nvshmem_free");
  host_barrier_all_blocking();  // every PE is done with the object
  std::lock_guard<std::mutex> lk(r.mu);
  if (r.heap->release(ptr) != HEAP_OK) ERROR_PRINT("nvshmem_free: %p was not returned by a symmetric allocation", ptr);
}
void* nvshmem_ptr(const void* dest, int pe) {
  if (!is_initialized()) return nullptr;
  return rt().heap->translate(dest, pe);
}
void* nvshmemx_mc_ptr(nvshmem_team_t team, const void* ptr) {
  if (!is_initialized()) return nullptr;
  Team* t = team_get(team);
  Runtime& r = rt();
  if (!t || !t->nvls || !t->mc_base || !r.heap->contains(ptr)) return nullptr;
  const size_t off = (size_t)((const char*)ptr - r.heap->base());
  return off < t->mc_bytes ? t->mc_base + off : nullptr;
}
void nvshmemx_b200_release_multicast(void) {
  if (!is_initialized()) return;
  Runtime& r = rt();
  r.heap->release_multicast_local();
  r.dstate.mc_base = 0;
  r.dstate.nvls_world = 0;
  teams_refresh_nvls(r);
  push_device_state();
}
// Local buffer registration matters most to NIC transports; with load/store peers every device buffer is
// already usable as a local source or target.
// What registration does here: it keeps a sorted table of the ranges (double registration and unknown
// unregistration are errors, as in the reference), and page-locks pageable host memory so that stream-ordered
// puts and gets with it as the local side run asynchronously.  (reference: src/host/mem/mem.cpp:32-443)
namespace {
struct LocalRange {
  char* base;
  size_t bytes;
  bool pinned_here;
};
std::vector<LocalRange> g_local_ranges;  // sorted by base; guarded by g_local_mu
std::mutex g_local_mu;
}  // namespace
int nvshmemx_buffer_register(void* addr, size_t length) {
  if (!addr || length == 0) return NVSHMEMX_ERROR_INVALID_VALUE;
  std::lock_guard<std::mutex> lk(g_local_mu);
  char* b = (char*)addr;
  auto it = std::lower_bound(g_local_ranges.begin(), g_local_ranges.end(), b, [](const LocalRange& r, char* p) { return r.base < p; });
  if (it != g_local_ranges.end() && it->base < b + length) return NVSHMEMX_ERROR_INVALID_VALUE;        // overlaps the next range
  if (it != g_local_ranges.begin() && (it - 1)->base + (it - 1)->bytes > b) return NVSHMEMX_ERROR_INVALID_VALUE;  // overlaps the previous one
  bool pinned = false;
  if (rt().have_gpu) {
    cudaPointerAttributes attr{};
    const bool known = cudaPointerGetAttributes(&attr, addr) == cudaSuccess && attr.type != cudaMemoryTypeUnregistered;
    cudaGetLastError();
    if (!known) {
      if (cudaHostRegister(addr, length, cudaHostRegisterPortable) != cudaSuccess) {
        cudaGetLastError();
        return NVSHMEMX_ERROR_INTERNAL;
      }
      pinned = true;
    }
  }
  g_local_ranges.insert(it, LocalRange{b, length, pinned});
  return NVSHMEMX_SUCCESS;
}
int nvshmemx_buffer_unregister(void* addr) {
  std::lock_guard<std::mutex> lk(g_local_mu);
  for (auto it = g_local_ranges.begin(); it != g_local_ranges.end(); ++it)
    if (it->base == (char*)addr) {
      if (it->pinned_here) cudaHostUnregister(addr);
      g_local_ranges.erase(it);
      return NVSHMEMX_SUCCESS;
    }
  return NVSHMEMX_ERROR_INVALID_VALUE;
}
void nvshmemx_buffer_unregister_all(void) {
  std::lock_guard<std::mutex> lk(g_local_mu);
  for (auto& r : g_local_ranges)
    if (r.pinned_here) cudaHostUnregister(r.base);
  g_local_ranges.clear();
}
// Maps a caller-owned VMM allocation into the symmetric heap (collective; same size on every PE) and returns
// its symmetric address; the caller's own mapping stays valid and aliases it.
static void republish_heap(Runtime& r) {
  r.dstate.heap_size = r.heap->backed();
  r.dstate.mc_base = (uint64_t)r.heap->mc_base();
  r.dstate.nvls_world = r.heap->mc_base() != nullptr;
  teams_refresh_nvls(r);
  push_device_state();
}
void* nvshmemx_buffer_register_symmetric(void* buf_ptr, size_t size, int flags) {
  (void)flags;
  if (!ready("nvshmemx_buffer_register_symmetric")) return nullptr;
  Runtime& r = rt();
  void* mapped = nullptr;
  {
    std::lock_guard<std::mutex> lk(r.mu);
    if (!r.have_gpu) {
      ERROR_PRINT("nvshmemx_buffer_register_symmetric needs the GPU heap back end");
      return nullptr;
    }
    int st = r.heap->attach_external(buf_ptr, size, &mapped);
    if (st != HEAP_OK) {
      ERROR_PRINT("nvshmemx_buffer_register_symmetric(%p, %zu) failed (status %d; sizes are multiples of %zu bytes)", buf_ptr, size, st, r.heap->granule());
      return nullptr;
    }
    republish_heap(r);
  }
  host_barrier_all_blocking();
  return mapped;
}
int nvshmemx_buffer_unregister_symmetric(void* mmap_ptr, size_t size) {
  if (!ready("nvshmemx_buffer_unregister_symmetric")) return NVSHMEMX_ERROR_INVALID_VALUE;
  Runtime& r = rt();
  host_barrier_all_blocking();
  std::lock_guard<std::mutex> lk(r.mu);
  int st = r.heap->detach_external(mmap_ptr, size);
  if (st != HEAP_OK) return NVSHMEMX_ERROR_INVALID_VALUE;
  republish_heap(r);
  return NVSHMEMX_SUCCESS;
}

// ------------------------------------------------------------------ teams
int nvshmem_team_my_pe(nvshmem_team_t team) {
  Team* t = team_get(team);
  return t ? t->my_pe : -1;
}
int nvshmem_team_n_pes(nvshmem_team_t team) {
  Team* t = team_get(team);
  return t && t->my_pe >= 0 ? t->size : -1;
}
void nvshmem_team_get_config(nvshmem_team_t team, nvshmem_team_config_t* config) {
  Team* t = team_get(team);
  if (!t || !config) return;
  config->version = (2 << 16) + (int)sizeof(nvshmem_team_config_t);
  config->num_contexts = t->num_contexts;
  config->uniqueid = t->uniqueid;
}
int nvshmem_team_translate_pe(nvshmem_team_t s, int pe, nvshmem_team_t d) { return team_translate_pe(s, pe, d); }
int nvshmem_team_split_strided(nvshmem_team_t parent, int start, int stride, int size, const nvshmem_team_config_t* config, long, nvshmem_team_t* new_team) {
  if (!ready("nvshmem_team_split_strided") || !new_team) return 1;
  std::lock_guard<std::mutex> lk(rt().mu);
  int nt = NVSHMEM_TEAM_INVALID;
  int st = team_split_strided(parent, start, stride, size, config ? config->uniqueid : 0, config ? config->num_contexts : 0, &nt);
  *new_team = nt;
  return st;
}
int nvshmem_team_split_2d(nvshmem_team_t parent, int xrange, const nvshmem_team_config_t*, long, nvshmem_team_t* xteam, const nvshmem_team_config_t*, long,
                          nvshmem_team_t* yteam) {
  if (!ready("nvshmem_team_split_2d") || !xteam || !yteam) return 1;
  std::lock_guard<std::mutex> lk(rt().mu);
  return team_split_2d(parent, xrange, xteam, yteam);
}
void nvshmem_team_destroy(nvshmem_team_t team) {
  if (!ready("nvshmem_team_destroy")) return;
  std::lock_guard<std::mutex> lk(rt().mu);
  team_destroy(team);
}
int nvshmemx_team_get_uniqueid(nvshmemx_team_uniqueid_t* uniqueid) {
  if (!uniqueid) return 1;
  static uint64_t counter = 0;
  *uniqueid = ((uint64_t)rt().mype << 48) ^ ((uint64_t)getpid() << 20) ^ ++counter ^ 0xB200B200ull << 8;
  return 0;
}
int nvshmemx_team_init(nvshmem_team_t* team, nvshmem_team_config_t* config, long, int npes, int pe_idx_in_team) {
  // Collective over the world: members pass their index and the team size, every
  // other PE passes npes = 0 (with the same unique id in `config`).  The member list is
  // assembled from an allgather, so no PE has to know the others beforehand.
  if (!ready("nvshmemx_team_init") || !team || !config) return 1;
  Runtime& r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  struct Entry { uint64_t id; int32_t idx; int32_t npes; } mine{config->uniqueid, pe_idx_in_team, npes};
  std::vector<Entry> all(r.npes);
  if (r.boot.allgather(&mine, all.data(), sizeof(Entry), &r.boot) != 0) return 1;
  int size = 0;
  for (auto& e : all)
    if (e.id == config->uniqueid) size = std::max(size, e.npes);
  *team = NVSHMEM_TEAM_INVALID;
  if (size <= 0) return 1;
  std::vector<int> members(size, -1);
  for (int pe = 0; pe < r.npes; ++pe)
    if (all[pe].id == config->uniqueid && all[pe].npes == size && all[pe].idx >= 0 && all[pe].idx < size) members[all[pe].idx] = pe;
  for (int m : members)
    if (m < 0) return 1;
  int nt = NVSHMEM_TEAM_INVALID;
  int st = team_create_from_members(NVSHMEM_TEAM_WORLD, members, config->uniqueid, &nt);
  *team = nt;
  return st;
}

// ------------------------------------------------------------------ ordering / signals
void nvshmem_quiet(void) {
  if (!ready("nvshmem_quiet")) return;
  Runtime& r = rt();
  NvtxRange nvtx(NVTX_MEMORDER, "nvshmem_quiet");
  if (!r.have_gpu) {
    __atomic_thread_fence(__ATOMIC_SEQ_CST);
    return;
  }
  for (size_t i = 0; i < r.peer_streams.size(); ++i)
    if (r.peer_stream_used[i]) {
      cudaStreamSynchronize(r.peer_streams[i]);
      r.peer_stream_used[i] = false;
    }
  cudaStreamSynchronize(r.stream);
}
void nvshmem_fence(void) { nvshmem_quiet(); }
void nvshmemx_quiet_on_stream(cudaStream_t stream) {
  if (!ready("nvshmemx_quiet_on_stream")) return;
  Runtime& r = rt();
  if (!r.have_gpu) return;
  NvtxRange nvtx(NVTX_QUIET_ON_STREAM, "nvshmemx_quiet_on_stream");
  for (size_t i = 0; i < r.peer_streams.size(); ++i)
    if (r.peer_stream_used[i]) {
      cudaEventRecord(r.ev_a, r.peer_streams[i]);
      cudaStreamWaitEvent(stream, r.ev_a, 0);
    }
  p2p_quiet_on_stream(stream);
}
uint64_t nvshmem_signal_fetch(uint64_t* sig_addr) {
  if (!ready("nvshmem_signal_fetch")) return 0;
  Runtime& r = rt();
  uint64_t v = 0;
  if (!r.have_gpu) return __atomic_load_n(sig_addr, __ATOMIC_ACQUIRE);
  cudaMemcpy(&v, sig_addr, sizeof(v), cudaMemcpyDeviceToHost);
  return v;
}
void nvshmemx_signal_op_on_stream(uint64_t* sig_addr, uint64_t signal, int sig_op, int pe, cudaStream_t stream) {
  if (ready("nvshmemx_signal_op_on_stream")) signal_on_stream(sig_addr, signal, sig_op, pe, stream);
}
void nvshmemx_signal_op(uint64_t* sig_addr, uint64_t signal, int sig_op, int pe) {
  if (!ready("nvshmemx_signal_op")) return;
  Runtime& r = rt();
  signal_on_stream(sig_addr, signal, sig_op, pe, r.stream);
  if (r.have_gpu) cudaStreamSynchronize(r.stream);
}
void nvshmemx_signal_wait_until_on_stream(uint64_t* sig_addr, int cmp, uint64_t cmp_value, cudaStream_t stream) {
  if (ready("nvshmemx_signal_wait_until_on_stream")) wait_on_stream(sig_addr, cmp, cmp_value, 8, false, stream);
}

// ------------------------------------------------------------------ untyped RMA
void nvshmem_putmem(void* d, const void* s, size_t n, int pe) { rma(d, s, n, pe, true, COPY_BLOCKING, 0, "nvshmem_putmem"); }
void nvshmem_getmem(void* d, const void* s, size_t n, int pe) { rma(d, s, n, pe, false, COPY_BLOCKING, 0, "nvshmem_getmem"); }
void nvshmem_putmem_nbi(void* d, const void* s, size_t n, int pe) { rma(d, s, n, pe, true, COPY_NBI, 0, "nvshmem_putmem_nbi"); }
void nvshmem_getmem_nbi(void* d, const void* s, size_t n, int pe) { rma(d, s, n, pe, false, COPY_NBI, 0, "nvshmem_getmem_nbi"); }
void nvshmemx_putmem_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n, pe, true, COPY_STREAM, st, "nvshmemx_putmem_on_stream"); }
void nvshmemx_getmem_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n, pe, false, COPY_STREAM, st, "nvshmemx_getmem_on_stream"); }
void nvshmemx_putmem_nbi_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n, pe, true, COPY_STREAM, st, "nvshmemx_putmem_nbi_on_stream"); }
void nvshmemx_getmem_nbi_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n, pe, false, COPY_STREAM, st, "nvshmemx_getmem_nbi_on_stream"); }
void nvshmemx_putmem_signal_on_stream(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) {
  rma(d, s, n, pe, true, COPY_STREAM, st, "nvshmemx_putmem_signal_on_stream");
  if (is_initialized()) signal_on_stream(sig, v, op, pe, st);
}
void nvshmemx_putmem_signal_nbi_on_stream(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) {
  nvshmemx_putmem_signal_on_stream(d, s, n, sig, v, op, pe, st);
}

// ------------------------------------------------------------------ typed RMA
#define BSHMEM_DEF_RMA(N, T)                                                                                                            \
  void nvshmem_##N##_p(T* dest, const T value, int pe) { rma(dest, &value, sizeof(T), pe, true, COPY_BLOCKING, 0, "nvshmem_" #N "_p"); } \
  T nvshmem_##N##_g(const T* src, int pe) {                                                                                             \
    T v;                                                                                                                                \
    memset(&v, 0, sizeof(T));                                                                                                           \
    rma(&v, src, sizeof(T), pe, false, COPY_BLOCKING, 0, "nvshmem_" #N "_g");                                                           \
    return v;                                                                                                                           \
  }                                                                                                                                     \
  void nvshmem_##N##_put(T* d, const T* s, size_t n, int pe) { rma(d, s, n * sizeof(T), pe, true, COPY_BLOCKING, 0, "nvshmem_" #N "_put"); } \
  void nvshmem_##N##_get(T* d, const T* s, size_t n, int pe) { rma(d, s, n * sizeof(T), pe, false, COPY_BLOCKING, 0, "nvshmem_" #N "_get"); } \
  void nvshmem_##N##_put_nbi(T* d, const T* s, size_t n, int pe) { rma(d, s, n * sizeof(T), pe, true, COPY_NBI, 0, "nvshmem_" #N "_put_nbi"); } \
  void nvshmem_##N##_get_nbi(T* d, const T* s, size_t n, int pe) { rma(d, s, n * sizeof(T), pe, false, COPY_NBI, 0, "nvshmem_" #N "_get_nbi"); } \
  void nvshmem_##N##_iput(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { rma_strided(d, s, dst, sst, n, sizeof(T), pe, true, COPY_BLOCKING, 0, "nvshmem_" #N "_iput"); } \
  void nvshmem_##N##_iget(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { rma_strided(d, s, dst, sst, n, sizeof(T), pe, false, COPY_BLOCKING, 0, "nvshmem_" #N "_iget"); } \
  void nvshmemx_##N##_p_on_stream(T* dest, const T value, int pe, cudaStream_t st) { rma(dest, &value, sizeof(T), pe, true, COPY_STREAM, st, "nvshmemx_" #N "_p_on_stream"); } \
  T nvshmemx_##N##_g_on_stream(const T* src, int pe, cudaStream_t st) {                                                                 \
    T v;                                                                                                                                \
    memset(&v, 0, sizeof(T));                                                                                                           \
    rma(&v, src, sizeof(T), pe, false, COPY_STREAM, st, "nvshmemx_" #N "_g_on_stream");                                                 \
    if (rt().have_gpu) cudaStreamSynchronize(st);                                                                                       \
    return v;                                                                                                                           \
  }                                                                                                                                     \
  void nvshmemx_##N##_put_on_stream(T* d, const T* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * sizeof(T), pe, true, COPY_STREAM, st, "nvshmemx_" #N "_put_on_stream"); } \
  void nvshmemx_##N##_get_on_stream(T* d, const T* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * sizeof(T), pe, false, COPY_STREAM, st, "nvshmemx_" #N "_get_on_stream"); } \
  void nvshmemx_##N##_put_nbi_on_stream(T* d, const T* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * sizeof(T), pe, true, COPY_STREAM, st, "nvshmemx_" #N "_put_nbi_on_stream"); } \
  void nvshmemx_##N##_get_nbi_on_stream(T* d, const T* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * sizeof(T), pe, false, COPY_STREAM, st, "nvshmemx_" #N "_get_nbi_on_stream"); } \
  void nvshmemx_##N##_iput_on_stream(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe, cudaStream_t st) { rma_strided(d, s, dst, sst, n, sizeof(T), pe, true, COPY_STREAM, st, "nvshmemx_" #N "_iput_on_stream"); } \
  void nvshmemx_##N##_iget_on_stream(T* d, const T* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe, cudaStream_t st) { rma_strided(d, s, dst, sst, n, sizeof(T), pe, false, COPY_STREAM, st, "nvshmemx_" #N "_iget_on_stream"); } \
  void nvshmemx_##N##_put_signal_on_stream(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) { nvshmemx_putmem_signal_on_stream(d, s, n * sizeof(T), sig, v, op, pe, st); } \
  void nvshmemx_##N##_put_signal_nbi_on_stream(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) { nvshmemx_putmem_signal_on_stream(d, s, n * sizeof(T), sig, v, op, pe, st); }
BSHMEM_RMA_TYPES(BSHMEM_DEF_RMA)
#undef BSHMEM_DEF_RMA

#define BSHMEM_DEF_SIZED(BITS, T)                                                                                                       \
  void nvshmem_put##BITS(void* d, const void* s, size_t n, int pe) { rma(d, s, n * (BITS / 8), pe, true, COPY_BLOCKING, 0, "nvshmem_put" #BITS); } \
  void nvshmem_get##BITS(void* d, const void* s, size_t n, int pe) { rma(d, s, n * (BITS / 8), pe, false, COPY_BLOCKING, 0, "nvshmem_get" #BITS); } \
  void nvshmem_put##BITS##_nbi(void* d, const void* s, size_t n, int pe) { rma(d, s, n * (BITS / 8), pe, true, COPY_NBI, 0, "nvshmem_put" #BITS "_nbi"); } \
  void nvshmem_get##BITS##_nbi(void* d, const void* s, size_t n, int pe) { rma(d, s, n * (BITS / 8), pe, false, COPY_NBI, 0, "nvshmem_get" #BITS "_nbi"); } \
  void nvshmem_iput##BITS(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { rma_strided(d, s, dst, sst, n, BITS / 8, pe, true, COPY_BLOCKING, 0, "nvshmem_iput" #BITS); } \
  void nvshmem_iget##BITS(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe) { rma_strided(d, s, dst, sst, n, BITS / 8, pe, false, COPY_BLOCKING, 0, "nvshmem_iget" #BITS); } \
  void nvshmemx_put##BITS##_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * (BITS / 8), pe, true, COPY_STREAM, st, "nvshmemx_put" #BITS "_on_stream"); } \
  void nvshmemx_get##BITS##_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * (BITS / 8), pe, false, COPY_STREAM, st, "nvshmemx_get" #BITS "_on_stream"); } \
  void nvshmemx_put##BITS##_signal_on_stream(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) { nvshmemx_putmem_signal_on_stream(d, s, n * (BITS / 8), sig, v, op, pe, st); }
BSHMEM_SIZES(BSHMEM_DEF_SIZED)
#undef BSHMEM_DEF_SIZED
#define BSHMEM_DEF_SIZED_MORE(BITS, T)                                                                                                   \
  void nvshmemx_put##BITS##_signal_nbi_on_stream(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe, cudaStream_t st) { nvshmemx_putmem_signal_on_stream(d, s, n * (BITS / 8), sig, v, op, pe, st); } \
  void nvshmemx_put##BITS##_nbi_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * (BITS / 8), pe, true, COPY_STREAM, st, "nvshmemx_put" #BITS "_nbi_on_stream"); } \
  void nvshmemx_get##BITS##_nbi_on_stream(void* d, const void* s, size_t n, int pe, cudaStream_t st) { rma(d, s, n * (BITS / 8), pe, false, COPY_STREAM, st, "nvshmemx_get" #BITS "_nbi_on_stream"); } \
  void nvshmemx_iput##BITS##_on_stream(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe, cudaStream_t st) { rma_strided(d, s, dst, sst, n, BITS / 8, pe, true, COPY_STREAM, st, "nvshmemx_iput" #BITS "_on_stream"); } \
  void nvshmemx_iget##BITS##_on_stream(void* d, const void* s, ptrdiff_t dst, ptrdiff_t sst, size_t n, int pe, cudaStream_t st) { rma_strided(d, s, dst, sst, n, BITS / 8, pe, false, COPY_STREAM, st, "nvshmemx_iget" #BITS "_on_stream"); }
BSHMEM_SIZES(BSHMEM_DEF_SIZED_MORE)
#undef BSHMEM_DEF_SIZED_MORE

// Queue-pair handles: one path to every peer, so every handle is the default one.
int nvshmemx_qp_create(int num_qps, nvshmemx_qp_handle_t** out_qp_array) {
  if (num_qps <= 0 || !out_qp_array) return NVSHMEMX_ERROR_INVALID_VALUE;
  nvshmemx_qp_handle_t* h = (nvshmemx_qp_handle_t*)malloc(sizeof(nvshmemx_qp_handle_t) * (size_t)num_qps);
  if (!h) return NVSHMEMX_ERROR_OUT_OF_MEMORY;
  for (int i = 0; i < num_qps; ++i) h[i] = NVSHMEMX_QP_DEFAULT;
  *out_qp_array = h;
  return NVSHMEMX_SUCCESS;
}
int nvshmemx_set_attr_mpi_comm_args(void* mpi_comm, nvshmemx_init_attr_t* attr) {
  if (!attr) return NVSHMEMX_ERROR_INVALID_VALUE;
  attr->mpi_comm = mpi_comm;  // recorded; initialising with it is refused (no MPI bootstrap is built)
  return NVSHMEMX_SUCCESS;
}

// ------------------------------------------------------------------ on-stream waits
#define BSHMEM_DEF_WAIT(N, T)                                                                                                           \
  void nvshmemx_##N##_wait_until_on_stream(T* ivar, int cmp, T v, cudaStream_t s) {                                                     \
    if (ready("nvshmemx_" #N "_wait_until_on_stream")) wait_on_stream(ivar, cmp, (uint64_t)v, (int)sizeof(T), std::is_signed<T>::value, s); \
  }                                                                                                                                     \
  void nvshmemx_##N##_wait_until_all_on_stream(T* ivars, size_t n, const int* status, int cmp, T v, cudaStream_t s) { wait_all_impl<T>(ivars, n, status, cmp, nullptr, v, s); } \
  void nvshmemx_##N##_wait_until_all_vector_on_stream(T* ivars, size_t n, const int* status, int cmp, T* vs, cudaStream_t s) { wait_all_impl<T>(ivars, n, status, cmp, vs, (T)0, s); }
BSHMEM_WAIT_TYPES(BSHMEM_DEF_WAIT)
#undef BSHMEM_DEF_WAIT

// ------------------------------------------------------------------ host atomics
#define BSHMEM_DEF_AMO_STD(N, T)                                                                                                        \
  void nvshmem_##N##_atomic_inc(T* t, int pe) { T one = 1; host_amo(AMO_ADD, t, &one, nullptr, sizeof(T), pe, nullptr); }               \
  T nvshmem_##N##_atomic_fetch_inc(T* t, int pe) { T one = 1, old = 0; host_amo(AMO_FETCH_ADD, t, &one, nullptr, sizeof(T), pe, &old); return old; } \
  void nvshmem_##N##_atomic_add(T* t, T v, int pe) { host_amo(AMO_ADD, t, &v, nullptr, sizeof(T), pe, nullptr); }                       \
  T nvshmem_##N##_atomic_fetch_add(T* t, T v, int pe) { T old = 0; host_amo(AMO_FETCH_ADD, t, &v, nullptr, sizeof(T), pe, &old); return old; } \
  T nvshmem_##N##_atomic_compare_swap(T* t, T c, T v, int pe) { T old = 0; host_amo(AMO_CAS, t, &v, &c, sizeof(T), pe, &old); return old; }
#define BSHMEM_DEF_AMO_EXT(N, T)                                                                                                        \
  T nvshmem_##N##_atomic_fetch(const T* t, int pe) { T old = 0; host_amo(AMO_FETCH, (void*)t, nullptr, nullptr, sizeof(T), pe, &old); return old; } \
  void nvshmem_##N##_atomic_set(T* t, T v, int pe) { host_amo(AMO_SWAP, t, &v, nullptr, sizeof(T), pe, nullptr); }                      \
  T nvshmem_##N##_atomic_swap(T* t, T v, int pe) { T old = 0; host_amo(AMO_SWAP, t, &v, nullptr, sizeof(T), pe, &old); return old; }
#define BSHMEM_DEF_AMO_BIT(N, T)                                                                                                        \
  void nvshmem_##N##_atomic_and(T* t, T v, int pe) { host_amo(AMO_AND, t, &v, nullptr, sizeof(T), pe, nullptr); }                       \
  T nvshmem_##N##_atomic_fetch_and(T* t, T v, int pe) { T old = 0; host_amo(AMO_AND, t, &v, nullptr, sizeof(T), pe, &old); return old; } \
  void nvshmem_##N##_atomic_or(T* t, T v, int pe) { host_amo(AMO_OR, t, &v, nullptr, sizeof(T), pe, nullptr); }                         \
  T nvshmem_##N##_atomic_fetch_or(T* t, T v, int pe) { T old = 0; host_amo(AMO_OR, t, &v, nullptr, sizeof(T), pe, &old); return old; }  \
  void nvshmem_##N##_atomic_xor(T* t, T v, int pe) { host_amo(AMO_XOR, t, &v, nullptr, sizeof(T), pe, nullptr); }                       \
  T nvshmem_##N##_atomic_fetch_xor(T* t, T v, int pe) { T old = 0; host_amo(AMO_XOR, t, &v, nullptr, sizeof(T), pe, &old); return old; }
BSHMEM_STANDARD_AMO_TYPES(BSHMEM_DEF_AMO_STD)
BSHMEM_EXTENDED_AMO_TYPES(BSHMEM_DEF_AMO_EXT)
BSHMEM_BITWISE_AMO_TYPES(BSHMEM_DEF_AMO_BIT)
#undef BSHMEM_DEF_AMO_STD
#undef BSHMEM_DEF_AMO_EXT
#undef BSHMEM_DEF_AMO_BIT

// ------------------------------------------------------------------ collectives
void nvshmem_barrier_all(void) {
  if (ready("nvshmem_barrier_all")) host_barrier_all_blocking();
}
int nvshmem_barrier(nvshmem_team_t team) {
  if (!ready("nvshmem_barrier")) return 1;
  nvshmem_quiet();
  return host_barrier_team(team, rt().stream, true);
}
void nvshmem_sync_all(void) {
  if (ready("nvshmem_sync_all")) host_sync_team(0, rt().stream, true);
}
int nvshmem_team_sync(nvshmem_team_t team) {
  if (!ready("nvshmem_team_sync")) return 1;
  return host_sync_team(team, rt().stream, true);
}
void nvshmemx_barrier_all_on_stream(cudaStream_t s) {
  if (ready("nvshmemx_barrier_all_on_stream")) host_barrier_team(0, s, false);
}
int nvshmemx_barrier_on_stream(nvshmem_team_t team, cudaStream_t s) {
  if (!ready("nvshmemx_barrier_on_stream")) return 1;
  return host_barrier_team(team, s, false);
}
void nvshmemx_sync_all_on_stream(cudaStream_t s) {
  if (ready("nvshmemx_sync_all_on_stream")) host_sync_team(0, s, false);
}
int nvshmemx_team_sync_on_stream(nvshmem_team_t team, cudaStream_t s) {
  if (!ready("nvshmemx_team_sync_on_stream")) return 1;
  return host_sync_team(team, s, false);
}
int nvshmemx_alltoallmem_on_stream(nvshmem_team_t team, void* d, const void* s, size_t bytes, cudaStream_t st) { return coll_alltoall_on_stream(team, d, s, bytes, st); }
int nvshmemx_fcollectmem_on_stream(nvshmem_team_t team, void* d, const void* s, size_t bytes, cudaStream_t st) { return coll_fcollect_on_stream(team, d, s, bytes, st); }
int nvshmemx_broadcastmem_on_stream(nvshmem_team_t team, void* d, const void* s, size_t bytes, int root, cudaStream_t st) { return coll_broadcast_on_stream(team, d, s, bytes, root, st); }
int nvshmem_alltoallmem(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return coll_finish(coll_alltoall_on_stream(team, d, s, bytes, rt().stream), rt().stream); }
int nvshmem_fcollectmem(nvshmem_team_t team, void* d, const void* s, size_t bytes) { return coll_finish(coll_fcollect_on_stream(team, d, s, bytes, rt().stream), rt().stream); }
int nvshmem_broadcastmem(nvshmem_team_t team, void* d, const void* s, size_t bytes, int root) { return coll_finish(coll_broadcast_on_stream(team, d, s, bytes, root, rt().stream), rt().stream); }
int nvshmemx_double2_maxloc_reduce_on_stream(nvshmem_team_t team, double2* d, const double2* s, size_t nreduce, cudaStream_t st) {
  if (nreduce != 1) return NVSHMEMX_ERROR_INVALID_VALUE;
  return coll_maxloc_on_stream(team, d, s, st);
}

#define BSHMEM_DEF_COLL(N, T)                                                                                                           \
  int nvshmemx_##N##_alltoall_on_stream(nvshmem_team_t team, T* d, const T* s, size_t n, cudaStream_t st) { return coll_alltoall_on_stream(team, d, s, n * sizeof(T), st); } \
  int nvshmemx_##N##_fcollect_on_stream(nvshmem_team_t team, T* d, const T* s, size_t n, cudaStream_t st) { return coll_fcollect_on_stream(team, d, s, n * sizeof(T), st); } \
  int nvshmemx_##N##_broadcast_on_stream(nvshmem_team_t team, T* d, const T* s, size_t n, int root, cudaStream_t st) { return coll_broadcast_on_stream(team, d, s, n * sizeof(T), root, st); } \
  int nvshmem_##N##_alltoall(nvshmem_team_t team, T* d, const T* s, size_t n) { return nvshmem_alltoallmem(team, d, s, n * sizeof(T)); }   \
  int nvshmem_##N##_fcollect(nvshmem_team_t team, T* d, const T* s, size_t n) { return nvshmem_fcollectmem(team, d, s, n * sizeof(T)); }   \
  int nvshmem_##N##_broadcast(nvshmem_team_t team, T* d, const T* s, size_t n, int root) { return nvshmem_broadcastmem(team, d, s, n * sizeof(T), root); }
BSHMEM_RMA_TYPES(BSHMEM_DEF_COLL)
#undef BSHMEM_DEF_COLL

#define BSHMEM_DEF_REDUCE_OP(N, T, OPNAME, OPENUM)                                                                                      \
  int nvshmemx_##N##_##OPNAME##_reduce_on_stream(nvshmem_team_t team, T* d, const T* s, size_t n, cudaStream_t st) {                    \
    return coll_reduce_on_stream(team, d, s, n, DTypeOf<T>::value, OPENUM, st);                                                         \
  }                                                                                                                                     \
  int nvshmemx_##N##_##OPNAME##_reducescatter_on_stream(nvshmem_team_t team, T* d, const T* s, size_t n, cudaStream_t st) {             \
    return coll_reducescatter_on_stream(team, d, s, n, DTypeOf<T>::value, OPENUM, st);                                                  \
  }                                                                                                                                     \
  int nvshmem_##N##_##OPNAME##_reduce(nvshmem_team_t team, T* d, const T* s, size_t n) {                                                \
    return coll_finish(coll_reduce_on_stream(team, d, s, n, DTypeOf<T>::value, OPENUM, rt().stream), rt().stream);                      \
  }                                                                                                                                     \
  int nvshmem_##N##_##OPNAME##_reducescatter(nvshmem_team_t team, T* d, const T* s, size_t n) {                                         \
    return coll_finish(coll_reducescatter_on_stream(team, d, s, n, DTypeOf<T>::value, OPENUM, rt().stream), rt().stream);               \
  }
#define BSHMEM_DEF_BITWISE(N, T) BSHMEM_DEF_REDUCE_OP(N, T, and, 0) BSHMEM_DEF_REDUCE_OP(N, T, or, 1) BSHMEM_DEF_REDUCE_OP(N, T, xor, 2)
#define BSHMEM_DEF_ARITH(N, T) BSHMEM_DEF_REDUCE_OP(N, T, min, 3) BSHMEM_DEF_REDUCE_OP(N, T, max, 4) BSHMEM_DEF_REDUCE_OP(N, T, sum, 5) BSHMEM_DEF_REDUCE_OP(N, T, prod, 6)
BSHMEM_BITWISE_REDUCE_TYPES(BSHMEM_DEF_BITWISE)
BSHMEM_STANDARD_REDUCE_TYPES(BSHMEM_DEF_ARITH)
#undef BSHMEM_DEF_BITWISE
#undef BSHMEM_DEF_ARITH
#undef BSHMEM_DEF_REDUCE_OP

// ------------------------------------------------------------------ collective launch
// Kernels that call device collectives need all their CTAs resident at once:
// launch cooperatively on an internal high-priority stream, ordered with the
// caller's stream by events (reference: src/device/launch/collective_launch.cpp).
int nvshmemx_collective_launch_query_gridsize(const void* func, dim3 block, void**, size_t smem, int* gridsize) {
  if (!gridsize) return NVSHMEMX_ERROR_INVALID_VALUE;
  int per_sm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, func, (int)(block.x * block.y * block.z), smem) != cudaSuccess) return NVSHMEMX_ERROR_INTERNAL;
  *gridsize = per_sm * sms;
  return NVSHMEMX_SUCCESS;
}
int nvshmemx_collective_launch(const void* func, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t stream) {
  if (!ready("nvshmemx_collective_launch")) return NVSHMEMX_ERROR_INVALID_VALUE;
  Runtime& r = rt();
  NvtxRange nvtx(NVTX_LAUNCH, "nvshmemx_collective_launch");
  int max_grid = 0;
  if (nvshmemx_collective_launch_query_gridsize(func, block, args, smem, &max_grid) != NVSHMEMX_SUCCESS) return NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;
  if (grid.x == 0) grid = dim3(max_grid, 1, 1);
  if ((int)(grid.x * grid.y * grid.z) > max_grid) {
    ERROR_PRINT("collective launch: a grid of %u CTAs cannot be co-resident (limit %d)", grid.x * grid.y * grid.z, max_grid);
    return NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;
  }
  cudaEventRecord(r.ev_a, stream);
  cudaStreamWaitEvent(r.stream, r.ev_a, 0);
  cudaError_t e = cudaLaunchCooperativeKernel(func, grid, block, args, smem, r.stream);
  if (e != cudaSuccess) {
    ERROR_PRINT("collective launch failed: %s", cudaGetErrorString(e));
    return NVSHMEMX_ERROR_COLLECTIVE_LAUNCH_FAILED;
  }
  cudaEventRecord(r.ev_b, r.stream);
  cudaStreamWaitEvent(stream, r.ev_b, 0);
  return NVSHMEMX_SUCCESS;
}

// ------------------------------------------------------------------ library extensions
void nvshmemx_b200_set_ce_collectives(size_t min_bytes) { rt().ce_min_bytes = min_bytes; }
void nvshmemx_b200_module_sync(void) {
  if (is_initialized()) push_device_state();
}
uint32_t nvshmemx_b200_error_bits(void) {
  Runtime& r = rt();
  return r.status_host ? status_load(&r.status_host->error_bits) : 0;
}
void nvshmemx_b200_clear_errors(void) {
  Runtime& r = rt();
  if (!r.status_host) return;
  status_store(&r.status_host->error_bits, 0);
  status_store(&r.status_host->timeout_count, 0);
  r.reported_errors.store(0);
}
uint32_t nvshmemx_b200_timeout_info(bshmemi_status_t* out) {
  Runtime& r = rt();
  if (!r.status_host) return 0;
  if (out) memcpy(out, (const void*)r.status_host, sizeof(*out));
  return status_load(&r.status_host->timeout_count);
}
void nvshmemx_b200_set_wait_timeout_ms(long ms) {
  Runtime& r = rt();
  r.dstate.wait_timeout_ns = (uint64_t)ms * 1000000ull;
  if (is_initialized()) push_device_state();
}
const char* nvshmemx_b200_topology(void) {
  static std::string s;
  s = rt().topo.describe();
  return s.c_str();
}
uint64_t nvshmemx_b200_heap_info(int what) {
  Runtime& r = rt();
  if (!r.heap) return 0;
  switch (what) {
    case 0: return (uint64_t)r.heap->base();
    case 1: return r.heap->stride();
    case 2: return r.heap->backed();
    case 3: return (uint64_t)r.heap->mc_base();
    case 4: return (uint64_t)r.heap->chunks();
    case 5: return r.heap->allocator().bytes_in_use();
    case 6: return r.heap->allocator().history_digest();
    case 7: return r.have_gpu ? 1 : 0;
    case 8: return (uint64_t)(int64_t)r.device;  // CUDA device of this PE (-1 on the host back end)
    default: return 0;
  }
}
int nvshmemx_b200_reduce_on_stream(nvshmem_team_t team, void* d, const void* s, size_t n, int dtype, int op, int algo, cudaStream_t st) { return coll_reduce_on_stream(team, d, s, n, dtype, op, st, algo); }
int nvshmemx_b200_reducescatter_on_stream(nvshmem_team_t team, void* d, const void* s, size_t n, int dtype, int op, int algo, cudaStream_t st) { return coll_reducescatter_on_stream(team, d, s, n, dtype, op, st, algo); }
int nvshmemx_b200_fcollect_on_stream(nvshmem_team_t team, void* d, const void* s, size_t bytes, int algo, cudaStream_t st) { return coll_fcollect_on_stream(team, d, s, bytes, st, algo); }
int nvshmemx_b200_broadcast_on_stream(nvshmem_team_t team, void* d, const void* s, size_t bytes, int root, int algo, cudaStream_t st) { return coll_broadcast_on_stream(team, d, s, bytes, root, st, algo); }

}  // extern "C"
