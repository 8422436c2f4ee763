#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <sstream>

#include "../util/cuda_dl.h"
#include "../util/env.h"
#include "../util/log.h"
#include "../util/nvtx.h"
#include "runtime.h"
#include "../transport/transport.h"

namespace bshmem {

Runtime& rt() {
  static Runtime* r = new Runtime();  // never destroyed: device modules may unregister late
  return *r;
}

bool is_initialized() { return rt().init_status >= INIT_IS_INITIALIZED; }

std::string TopoRecord::describe() const {
  std::ostringstream os;
  os << device_count << "x " << name << " (sm_" << cc_major << cc_minor << ", " << sm_count << " SMs), PCI " << pci_bus_id
     << ", NVLink v" << nvlink_version << " x" << nvlink_links << (nvswitch ? " via NVSwitch" : "")
     << ", peers ld/st " << (all_peers_ldst ? "all" : "partial") << ", atomics " << (all_peers_atomics ? "all" : "partial")
     << ", multicast " << (multicast_supported ? "yes" : "no");
  return os.str();
}

int probe_topology(Runtime& r) {
  TopoRecord& t = r.topo;
  t.device = r.device;
  cudaGetDeviceCount(&t.device_count);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, r.device) != cudaSuccess) return ST_INTERNAL;
  t.name = prop.name;
  t.cc_major = prop.major;
  t.cc_minor = prop.minor;
  t.sm_count = prop.multiProcessorCount;
  char bus[32] = "";
  cudaDeviceGetPCIBusId(bus, sizeof(bus), r.device);
  t.pci_bus_id = bus;
  t.uuid.assign((const char*)&prop.uuid, 16);
  const CuTable* d = cu();
  if (d) {
    CUdevice dev;
    if (d->cuDeviceGet_(&dev, r.device) == CUDA_SUCCESS) {
      int v = 0;
      d->cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
      t.multicast_supported = v != 0;
      d->cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
      t.vmm_supported = v != 0;
      d->cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_CAN_USE_64_BIT_STREAM_MEM_OPS_V1, dev);
      t.stream_memops = v != 0;
    }
  }
  NvlinkInfo nv = nvml_probe_nvlink(bus);
  t.nvlink_links = nv.active_links;
  t.nvlink_version = nv.link_version;
  t.nvswitch = nv.all_links_to_switch;
  return ST_SUCCESS;
}

// Asks every transport which peers it reaches (the built-in P2P transport first, then a plugin named by
// NVSHMEM_REMOTE_TRANSPORT), records per PE the first transport that reaches it, and fills the reach bits that the
// rest of bring-up reads: bit 0 load/store, bit 1 native atomics, bit 2 same device
// (reference: src/host/transport/transport.cpp nvshmemi_transport_init + nvshmemi_setup_connections,
//  src/host/transport/p2p/p2p.cpp nvshmemt_p2p_can_reach_peer).
static int build_reach_map(Runtime& r) {
  TopoRecord& t = r.topo;
  t.reach.assign(r.npes, 0);
  if (r.transports.empty()) {
    bshmem_transport* p2p = nullptr;
    if (transport_p2p_init(&p2p) != 0) return ST_INTERNAL;
    r.transports.push_back(p2p);
    const std::string remote = options().REMOTE_TRANSPORT;
    if (!remote.empty() && remote != "none" && remote != "NONE") {
      bshmem_transport* extra = nullptr;
      if (transport_load_plugin(remote, &extra) != 0) return ST_NOT_SUPPORTED;
      r.transports.push_back(extra);
    }
  }
  r.transport_of_pe.assign(r.npes, -1);
  for (size_t ti = 0; ti < r.transports.size(); ++ti) {
    bshmem_transport* tr = r.transports[ti];
    tr->cap.assign(r.npes, 0);
    for (int pe = 0; pe < r.npes; ++pe) {
      uint32_t caps = 0;
      if (tr->ops.can_reach_peer(tr, &r.pe_info[r.mype], &r.pe_info[pe], r.device, &caps) != 0) caps = 0;
      tr->cap[pe] = caps;
      if (caps && r.transport_of_pe[pe] < 0) r.transport_of_pe[pe] = (int)ti;
    }
    if (tr->ops.connect_endpoints && !(tr->attr & TRANSPORT_ATTR_NO_ENDPOINTS)) {
      std::vector<int> mine;
      for (int pe = 0; pe < r.npes; ++pe)
        if (r.transport_of_pe[pe] == (int)ti) mine.push_back(pe);
      if (!mine.empty() && tr->ops.connect_endpoints(tr, mine.data(), (int)mine.size()) != 0) return ST_INTERNAL;
    }
    std::string info;
    if (tr->ops.show_info && tr->ops.show_info(tr, &info) == 0) INFO(SUB_TRANSPORT, "transport %zu: %s", ti, info.c_str());
  }
  for (int pe = 0; pe < r.npes; ++pe) {
    const int ti = r.transport_of_pe[pe];
    const uint32_t caps = ti >= 0 ? r.transports[ti]->cap[pe] : 0;
    uint8_t bits = 0;
    // Only the built-in transport gives GPU threads direct access; a peer reached by a plugin alone is not
    // load/store reachable and bring-up refuses it further down (no proxy path is built).
    if (ti == 0 && (caps & TRANSPORT_CAP_GPU_LD) && (caps & TRANSPORT_CAP_GPU_ST)) bits |= 1;
    if (ti == 0 && (caps & TRANSPORT_CAP_GPU_ATOMICS)) bits |= 2;
    if (caps & TRANSPORT_CAP_SAME_DEVICE) bits |= 4;
    t.reach[pe] = bits;
    if (!(bits & 1)) t.all_peers_ldst = false;
    if (!(bits & 2)) t.all_peers_atomics = false;
  }
  return ST_SUCCESS;
}

void push_pending_modules() {
  Runtime& r = rt();
  if (!r.modules_pending.load() || r.init_status < INIT_IS_INITIALIZED) return;
  push_device_state();
}

int push_device_state() {
  Runtime& r = rt();
  r.modules_pending.store(false);
  if (!r.have_gpu) return ST_SUCCESS;
  for (auto& m : r.modules) {
    void* addr = m.first();
    if (!addr) continue;
    cudaError_t e = cudaMemcpy(addr, &r.dstate, sizeof(r.dstate), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      ERROR_PRINT("copying the device state into module %s failed: %s", m.second.c_str(), cudaGetErrorString(e));
      return ST_INTERNAL;
    }
  }
  // Modules loaded through the driver API and announced with nvshmemx_cumodule_init / nvshmemx_culibrary_init.
  for (auto& m : r.driver_modules) {
    if (cudaMemcpy(m.second, &r.dstate, sizeof(r.dstate), cudaMemcpyHostToDevice) != cudaSuccess) {
      ERROR_PRINT("copying the device state into a driver-API module failed");
      return ST_INTERNAL;
    }
  }
  return ST_SUCCESS;
}

// ------------------------------------------------------------------ watchdog
// Replaces the reference's proxy thread for a load/store-only job: it services
// device-side nvshmem_global_exit and reports (or, when asked, acts on) device
// wait time-outs.  Device code never spins for ever, so the watchdog never has
// to kill the process to unblock a kernel
// (reference: src/host/proxy/proxy.cpp, minimal proxy, progress_timeout_polling).
static void watchdog_main(Runtime* r) {
  pthread_setname_np(pthread_self(), "bshmem-watchdog");
  while (!r->watchdog_stop.load()) {
    bshmemi_status_t* s = r->status_host;
    if (s) {
      uint32_t bits = status_load(&s->error_bits);
      uint32_t fresh = bits & ~r->reported_errors.load();
      if (fresh) {
        r->reported_errors.fetch_or(fresh);
        if (fresh & BSHMEM_ERR_WAIT_TIMEOUT)
          ERROR_PRINT("PE %d: a device-side wait timed out (where=%u addr=%#llx expected=%llu found=%llu); the kernel returned with an error status",
                      r->mype, s->timeout_where, (unsigned long long)s->timeout_addr, (unsigned long long)s->timeout_expected,
                      (unsigned long long)s->timeout_found);
        if (fresh & ~BSHMEM_ERR_WAIT_TIMEOUT & ~BSHMEM_ERR_GLOBAL_EXIT)
          ERROR_PRINT("PE %d: device code reported error bits %#x", r->mype, fresh);
        if ((fresh & BSHMEM_ERR_WAIT_TIMEOUT) && options().WATCHDOG_ABORT) {
          if (r->boot_live && r->boot.global_exit) r->boot.global_exit(-1, &r->boot);
          _exit(-1);
        }
      }
      if (status_load(&s->global_exit_req)) {
        int code = s->global_exit_code;
        INFO(SUB_INIT, "PE %d: device code called nvshmem_global_exit(%d)", r->mype, code);
        if (r->boot_live && r->boot.global_exit) r->boot.global_exit(code, &r->boot);
        _exit(code);
      }
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

void watchdog_start(Runtime& r) {
  if (options().DISABLE_WATCHDOG) return;
  r.watchdog_stop.store(false);
  r.watchdog = std::thread(watchdog_main, &r);
}

void watchdog_stop(Runtime& r) {
  r.watchdog_stop.store(true);
  if (r.watchdog.joinable()) r.watchdog.join();
}

// ------------------------------------------------------------------ init
// Share of the GPU's SMs that an MPS server grants this process, in percent; -1 when no MPS server serves it.
// A client of an MPS server sees the server's pipe directory (CUDA_MPS_PIPE_DIRECTORY, default /tmp/nvidia-mps) with
// its control file; CUDA_MPS_ACTIVE_THREAD_PERCENTAGE narrows the share (100 when it is not set).
// (reference: src/host/init/init.cu:724-947 decides LIMITED / FULL the same way: MPS present and the shares of the
// PEs on a GPU sum to at most 100.)
static int mps_share_of_this_process() {
  const char* dir = getenv("CUDA_MPS_PIPE_DIRECTORY");
  std::string control = std::string(dir && *dir ? dir : "/tmp/nvidia-mps") + "/control";
  if (access(control.c_str(), F_OK) != 0) return -1;
  const char* pct = getenv("CUDA_MPS_ACTIVE_THREAD_PERCENTAGE");
  if (!pct || !*pct) return 100;
  char* end = nullptr;
  double v = strtod(pct, &end);
  if (end == pct || v <= 0 || v > 100) return 100;
  return (int)(v + 0.999);
}

// Counts the PEs that share this PE's GPU and decides what they may do together.
static void classify_gpu_sharing(Runtime& r) {
  const PeInfo& me = r.pe_info[r.mype];
  int sharers = 0, share_sum = 0;
  bool all_mps = true;
  for (const PeInfo& p : r.pe_info) {
    if (p.host_hash != me.host_hash || memcmp(p.uuid, me.uuid, sizeof(me.uuid)) != 0) continue;
    ++sharers;
    if (p.mps_percent < 0) all_mps = false;
    else share_sum += p.mps_percent;
  }
  r.pes_on_my_gpu = sharers;
  const bool shares_fit = share_sum <= 100 || options().IGNORE_CUDA_MPS_ACTIVE_THREAD_PERCENTAGE;
  r.mpg_status = sharers <= 1 ? MPG_NONE : (all_mps && shares_fit) ? MPG_FULL : MPG_LIMITED;
  if (r.mpg_status == MPG_LIMITED)
    WARN("%d PEs share the GPU of PE %d and nothing guarantees that their kernels run at the same time (no MPS server, or shares above 100%%): "
               "host-initiated operations between them work; device code of one PE must not wait for device code of another "
               "(barriers, collectives and signal waits inside kernels)", sharers, r.mype);
  else if (r.mpg_status == MPG_FULL)
    INFO(SUB_INIT, "%d PEs share the GPU of PE %d under an MPS server with %d%% of the SMs between them", sharers, r.mype, share_sum);
}

static void print_options_if_asked(const Runtime& r) {
  const Options& o = options();
  if (o.VERSION && r.mype == 0) printf("%s version %d.%d.%d\n", BSHMEM_VENDOR_STRING, BSHMEM_MAJOR, BSHMEM_MINOR, BSHMEM_PATCH);
  if (o.INFO && r.mype == 0) {
    for (auto& i : options_describe(o)) {
      if (i.cat == OptCat::Hidden && !o.INFO_HIDDEN) continue;
      printf("%-40s %s%s\n", i.name, i.value.c_str(), i.set ? "  (set)" : "");
    }
  }
}

int runtime_init(const bshmem_uniqueid_t* id, int rank, int nranks, int device_hint, bool hostlib_only, int boot_mode) {
  Runtime& r = rt();
  if (r.init_status >= INIT_IS_INITIALIZED) return ST_SUCCESS;
  NvtxRange nvtx(NVTX_INIT, "nvshmem_init");
  std::vector<std::string> bad;
  Options tmp;
  if (options_init(&tmp, &bad) != 0) {
    for (auto& b : bad) ERROR_PRINT("invalid value in environment: %s", b.c_str());
    return ST_INVALID_VALUE;
  }
  options_reload();
  log_init();
  nvtx_init();
  const Options& o = options();
  r.hostlib_only = hostlib_only;
  if (o.DEBUG_ATTACH_DELAY > 0) {
    fprintf(stderr, "bshmem: pid %d waits %ld s for a debugger (NVSHMEM_DEBUG_ATTACH_DELAY)\n", (int)getpid(), o.DEBUG_ATTACH_DELAY);
    sleep((unsigned)o.DEBUG_ATTACH_DELAY);
  }
  {
    std::string kind = o.HEAP_KIND;
    std::transform(kind.begin(), kind.end(), kind.begin(), ::toupper);
    if (kind != "VIDMEM") {
      ERROR_PRINT("NVSHMEM_HEAP_KIND=%s: only VIDMEM is built (a heap in pinned host memory is not); NVSHMEM_HEAP_BACKEND=HOST gives a host-memory heap for runs without a GPU",
                  o.HEAP_KIND.c_str());
      return ST_NOT_SUPPORTED;
    }
  }

  int st = bootstrap_init(boot_mode, id, rank, nranks, &r.boot);
  if (st != BOOT_OK) {
    ERROR_PRINT("bootstrap failed: %s", bootstrap_strerror(st));
    return ST_INTERNAL;
  }
  r.boot_live = true;
  r.mype = r.boot.pg_rank;
  r.npes = r.boot.pg_size;
  r.mype_node = r.boot.mype_node;
  r.npes_node = r.boot.npes_node;
  r.init_status = INIT_IS_BOOTSTRAPPED;
  log_set_pe(r.mype);
  print_options_if_asked(r);
  log_process_diagnostics();

  // ---- which back end
  int ndev = 0;
  bool gpu = cu() != nullptr && cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
  std::string be = o.HEAP_BACKEND;
  std::transform(be.begin(), be.end(), be.begin(), ::toupper);
  if (o.DISABLE_CUDA_VMM && gpu && be != "HOST") {
    // The reference's alternative to VMM is one cudaMalloc per PE shared through CUDA IPC.  IPC mappings land at
    // addresses the driver picks, while this library's address translation relies on all PEs' heaps sitting at fixed
    // offsets of one reservation, so that heap is not built; a job that asks for it gets an error, not host memory.
    ERROR_PRINT("NVSHMEM_DISABLE_CUDA_VMM is set, but the GPU heap of this library needs CUDA virtual memory management (every sm_100 GPU has it); "
                "unset the variable, or set NVSHMEM_HEAP_BACKEND=HOST for a heap in host memory");
    return ST_NOT_SUPPORTED;
  }
  bool use_vmm = be == "VMM" || (be == "AUTO" && gpu);
  if (use_vmm && !gpu) {
    ERROR_PRINT("NVSHMEM_HEAP_BACKEND=VMM needs a CUDA device");
    return ST_GPU_NOT_SELECTED;
  }
  r.have_gpu = use_vmm;
  if (use_vmm) {
    if (device_hint >= 0) {
      r.device = device_hint;
    } else {
      // No device named: a process that already holds a CUDA context keeps its device; one that has not touched
      // CUDA yet gets the device of its rank on the node, which is what programs that call cudaSetDevice(mype_node)
      // after nvshmem_init() expect (reference: examples/ring-bcast.cu, init-then-select pattern).
      CUcontext ctx = nullptr;
      const bool has_ctx = cu()->cuCtxGetCurrent_(&ctx) == CUDA_SUCCESS && ctx != nullptr;
      if (!has_ctx) r.device = r.mype_node % ndev;
      else if (cudaGetDevice(&r.device) != cudaSuccess) r.device = 0;
    }
    if (cudaSetDevice(r.device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) {
      ERROR_PRINT("cannot select CUDA device %d", r.device);
      return ST_GPU_NOT_SELECTED;
    }
    log_set_device(r.device);
    if (o.CUDA_LIMIT_STACK_SIZE > 0 && cudaDeviceSetLimit(cudaLimitStackSize, o.CUDA_LIMIT_STACK_SIZE) != cudaSuccess)
      WARN("NVSHMEM_CUDA_LIMIT_STACK_SIZE=%zu was refused by the CUDA runtime", o.CUDA_LIMIT_STACK_SIZE);
    if (probe_topology(r) != ST_SUCCESS) return ST_INTERNAL;
  }

  // ---- who is where
  PeInfo mine{};
  mine.pid = (int32_t)getpid();
  mine.device = r.device;
  mine.host_hash = host_hash();
  strncpy(mine.pci_bus_id, r.topo.pci_bus_id.c_str(), sizeof(mine.pci_bus_id) - 1);
  if (r.topo.uuid.size() == 16) memcpy(mine.uuid, r.topo.uuid.data(), 16);
  else if (!use_vmm && o.TEST_FAKE_GPU >= 0) snprintf(mine.uuid, sizeof(mine.uuid), "fakegpu-%ld", o.TEST_FAKE_GPU);
  else snprintf(mine.uuid, sizeof(mine.uuid), "host-%d", r.mype);
  mine.mps_percent = mps_share_of_this_process();
  r.pe_info.resize(r.npes);
  if (r.boot.allgather(&mine, r.pe_info.data(), sizeof(PeInfo), &r.boot) != 0) return ST_INTERNAL;
  classify_gpu_sharing(r);
  if (use_vmm) {
    build_reach_map(r);
    if (!r.topo.all_peers_ldst) {
      ERROR_PRINT("PE %d cannot load/store to every peer; only NVLink/NVSwitch-connected jobs on one node are supported (no remote transport is built)", r.mype);
      return ST_NOT_SUPPORTED;
    }
    INFO(SUB_TOPO, "topology: %s", r.topo.describe().c_str());
  }

  // ---- heap
  size_t stride = o.MAX_MEMORY_PER_GPU, initial = o.SYMMETRIC_SIZE, gran = o.CUMEM_GRANULARITY;
  if (use_vmm) {
    r.heap = make_vmm_heap(!o.DISABLE_NVLS);
  } else {
    r.heap = make_host_heap();
    if (!o.CUMEM_GRANULARITY_set) gran = (size_t)1 << 20;
    if (!o.MAX_MEMORY_PER_GPU_set) stride = std::max<size_t>((size_t)4 << 30, initial * 4);
  }
  st = r.heap->init(&r.boot, r.device, stride, initial, gran);
  if (st != HEAP_OK) {
    ERROR_PRINT("symmetric heap (%s) initialisation failed with status %d", r.heap->kind(), st);
    return st == HEAP_ERR_OOM ? ST_OUT_OF_MEMORY : ST_INTERNAL;
  }

  // ---- status block + device state
  if (use_vmm) {
    if (cudaHostAlloc((void**)&r.status_host, sizeof(bshmemi_status_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return ST_OUT_OF_MEMORY;
    memset((void*)r.status_host, 0, sizeof(bshmemi_status_t));
    void* dptr = nullptr;
    cudaHostGetDevicePointer(&dptr, r.status_host, 0);
    r.dstate.status = (uint64_t)dptr;
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    cudaStreamCreateWithPriority(&r.stream, cudaStreamNonBlocking, greatest);
    r.peer_streams.resize((size_t)std::max<long>(1, std::min<long>(r.npes, o.MAX_PEER_STREAMS)));
    for (auto& s : r.peer_streams) cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    r.peer_stream_used.assign(r.peer_streams.size(), false);
    cudaEventCreateWithFlags(&r.ev_a, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&r.ev_b, cudaEventDisableTiming);
  } else {
    r.status_host = new bshmemi_status_t();
    memset((void*)r.status_host, 0, sizeof(bshmemi_status_t));
    r.dstate.status = (uint64_t)r.status_host;
  }
  bshmemi_state_t& d = r.dstate;
  d.version = (BSHMEM_MAJOR << 16) | (BSHMEM_MINOR << 8) | BSHMEM_PATCH;
  d.mype = r.mype;
  d.npes = r.npes;
  d.mype_node = r.mype_node;
  d.npes_node = r.npes_node;
  d.max_teams = r.max_teams = (int)std::max<long>(o.MAX_TEAMS, 8);
  d.job_connectivity = !use_vmm ? BSHMEM_JOB_HOST_ONLY : (r.topo.all_peers_atomics ? BSHMEM_JOB_GPU_LDST_ATOMICS : BSHMEM_JOB_GPU_LDST);
  d.heap_base = (uint64_t)r.heap->base();
  d.heap_stride = r.heap->stride();
  d.heap_size = r.heap->backed();
  d.mc_base = (uint64_t)r.heap->mc_base();
  d.nvls_world = r.heap->mc_base() != nullptr;
  d.wait_timeout_ns = (uint64_t)o.WAIT_TIMEOUT_MS * 1000000ull;
  d.reduce_algo = (int)o.REDUCE_ALGO;
  d.fcollect_algo = (int)o.FCOLLECT_ALGO;
  d.reducescatter_algo = (int)o.REDUCESCATTER_ALGO;
  d.bcast_algo = (int)o.BCAST_ALGO;
  d.sync_gpu_release = o.SYNC_GPU_SCOPE_RELEASE ? 1 : 0;
  d.barrier_dissem_kval = (int)std::max<long>(o.BARRIER_DISSEM_KVAL, 2);
  d.barrier_tg_dissem_kval = (int)std::max<long>(o.BARRIER_TG_DISSEM_KVAL, 2);
  d.bcast_tree_kval = (int)std::max<long>(o.BCAST_TREE_KVAL, 2);
  d.debug_checks = o.ENABLE_ERROR_CHECKS;
  r.ce_min_bytes = o.CE_COLLECTIVES_MIN_BYTES;
  d.reduce_nvls_threshold = o.REDUCE_NVLS_THRESHOLD;
  d.reduce_oneshot_threshold = o.REDUCE_ONESHOT_THRESHOLD;
  d.fcollect_ll_threshold = o.FCOLLECT_LL_THRESHOLD;
  d.ll128_threshold = o.FCOLLECT_LL128_THRESHOLD_set ? o.FCOLLECT_LL128_THRESHOLD : o.LL128_THRESHOLD;
  d.fcollect_nvls_threshold = o.FCOLLECT_NVLS_THRESHOLD;
  d.reducescatter_nvls_threshold = o.REDUCESCATTER_NVLS_THRESHOLD;

  // ---- teams (first symmetric allocation), then publish the state
  st = teams_init(r);
  if (st != ST_SUCCESS) return st;
  d.heap_size = r.heap->backed();
  st = push_device_state();
  if (st != ST_SUCCESS) return st;
  watchdog_start(r);
  r.init_status = INIT_IS_INITIALIZED;
  if (r.boot.barrier(&r.boot) != 0) return ST_INTERNAL;
  st = host_barrier_all_blocking();  // first cross-GPU traffic: proves the mappings
  if (st != ST_SUCCESS) return st;
  INFO(SUB_INIT, "PE %d of %d initialised: heap %s, %zu bytes backed, NVLS %s", r.mype, r.npes, r.heap->kind(), r.heap->backed(),
       d.nvls_world ? "on" : "off");
  return ST_SUCCESS;
}

int runtime_finalize() {
  Runtime& r = rt();
  if (r.init_status < INIT_IS_BOOTSTRAPPED) return ST_SUCCESS;
  NvtxRange nvtx(NVTX_INIT, "nvshmem_finalize");
  if (r.init_status >= INIT_IS_INITIALIZED) {
    if (r.have_gpu) cudaDeviceSynchronize();
    host_barrier_all_blocking();
    if (log_enabled(LOG_INFO, SUB_INIT))
      INFO(SUB_INIT, "PE %d counters: put %llu (%llu B) get %llu (%llu B) signal %llu coll %llu barrier %llu alloc %llu", r.mype,
           (unsigned long long)r.n_put, (unsigned long long)r.bytes_put, (unsigned long long)r.n_get, (unsigned long long)r.bytes_get,
           (unsigned long long)r.n_signal, (unsigned long long)r.n_coll, (unsigned long long)r.n_barrier, (unsigned long long)r.n_alloc);
  }
  watchdog_stop(r);
  teams_finalize(r);
  for (bshmem_transport* tr : r.transports) transport_destroy(tr);
  r.transports.clear();
  r.transport_of_pe.clear();
  if (r.have_gpu) {
    cudaDeviceSynchronize();
    if (r.stream) cudaStreamDestroy(r.stream);
    for (auto s : r.peer_streams) cudaStreamDestroy(s);
    r.peer_streams.clear();
    if (r.ev_a) cudaEventDestroy(r.ev_a);
    if (r.ev_b) cudaEventDestroy(r.ev_b);
    r.stream = nullptr;
    r.ev_a = r.ev_b = nullptr;
  }
  if (r.heap) {
    r.heap->finalize();
    r.heap.reset();
  }
  if (r.status_host) {
    if (r.have_gpu) cudaFreeHost((void*)r.status_host);
    else delete r.status_host;
    r.status_host = nullptr;
  }
  if (r.boot_live) {
    r.boot.barrier(&r.boot);
    r.boot.finalize(&r.boot);
    r.boot_live = false;
  }
  r.init_status = INIT_NOT_INITIALIZED;
  r.reported_errors.store(0);
  memset(&r.dstate, 0, sizeof(r.dstate));
  return ST_SUCCESS;
}

}  // namespace bshmem

extern "C" void bshmemi_register_module(void* (*getter)(), const char* name) {
  // Runs inside static initialisers of the registering library, possibly while that library's
  // device code is still being registered with the CUDA runtime: make no CUDA call here.  The
  // state reaches the module at initialisation, or at the next API call if the library was
  // loaded later (push_pending_modules).
  bshmem::Runtime& r = bshmem::rt();
  for (auto& m : r.modules)
    if (m.first == getter) return;
  r.modules.emplace_back(getter, name ? name : "?");
  r.modules_pending.store(true);
}
