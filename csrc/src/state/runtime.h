// Process-wide runtime of the host library: bootstrap handle, heap, topology
// record, team table, device-state mirror, internal streams and the watchdog
// thread.  Bring-up order (each step collective where noted):
//   options/log → bootstrap (collective) → device + topology probe → heap
//   (collective) → status block → team pool (collective) → device state push →
//   watchdog → first barrier (collective)
// (reference: src/host/init/init.cu, nvshmemi_common_init).
#pragma once
#include <cuda_runtime_api.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/bshmem/state.h"
#include "../bootstrap/bootstrap.h"
#include "../heap/heap.h"

namespace bshmem {

enum Status {  // public nvshmemx_status values
  ST_SUCCESS = 0,
  ST_INVALID_VALUE = 1,
  ST_OUT_OF_MEMORY = 2,
  ST_NOT_SUPPORTED = 3,
  ST_SYMMETRY = 4,
  ST_GPU_NOT_SELECTED = 5,
  ST_COLLECTIVE_LAUNCH_FAILED = 6,
  ST_INTERNAL = 7,
};

enum InitStatus { INIT_NOT_INITIALIZED = 0, INIT_IS_BOOTSTRAPPED = 1, INIT_IS_INITIALIZED = 2 };
// Several PEs on one GPU: NONE (one PE per GPU), LIMITED (their kernels may not run at the same time, so device code of
// one must not wait for device code of another), FULL (an MPS server gives each its own share of the SMs).
enum MpgStatus { MPG_NONE = 0, MPG_LIMITED = 1, MPG_FULL = 2 };

struct TopoRecord {
  int device = -1;
  int device_count = 0;
  std::string name, pci_bus_id, uuid;
  int cc_major = 0, cc_minor = 0, sm_count = 0;
  bool multicast_supported = false, vmm_supported = false, stream_memops = false;
  int nvlink_links = 0, nvlink_version = 0;
  bool nvswitch = false;
  bool all_peers_ldst = true, all_peers_atomics = true;
  std::vector<uint8_t> reach;  // per PE: bit0 ld/st, bit1 native atomics, bit2 same device
  std::string describe() const;
};

struct PeInfo {  // all-gathered at init
  int32_t pid;
  int32_t device;
  uint64_t host_hash;
  char pci_bus_id[32];
  char uuid[16];
  int32_t mps_percent;  // CUDA_MPS_ACTIVE_THREAD_PERCENTAGE of the process when an MPS server serves it, else -1
  int32_t reserved;
};

struct bshmem_transport;

struct Team {
  int idx = -1;
  int start = 0, stride = 1, size = 0, my_pe = -1;
  int parent = -1;
  std::vector<int> members;  // world PE of each member (always filled)
  bool strided = true;
  bool nvls = false;
  int mc_id = -1;               // the heap's handle of this team's own multicast window (-1: the world's, or none)
  char* mc_base = nullptr;      // multicast address of heap offset 0 for this team (null without NVLS)
  size_t mc_bytes = 0;          // bytes of the heap that the window covers
  int32_t* pe_of_dev = nullptr;  // device copy of `members` for non-strided teams
  uint64_t uniqueid = 0;
  int num_contexts = 0;
  std::vector<int> children;  // node sub-teams destroyed with this team
};

typedef void* (*StateAddrGetter)();

struct Runtime {
  std::mutex mu;  // serialises public entry points (thread level SERIALIZED)
  int init_status = INIT_NOT_INITIALIZED;
  int mpg_status = MPG_NONE;
  int pes_on_my_gpu = 1;
  bool hostlib_only = false;
  bshmem_bootstrap_handle_t boot{};
  bool boot_live = false;
  int mype = 0, npes = 1, mype_node = 0, npes_node = 1;
  int device = -1;
  bool have_gpu = false;
  TopoRecord topo;
  std::vector<PeInfo> pe_info;
  std::vector<bshmem_transport*> transports;   // [0] is the built-in load/store transport
  std::vector<int> transport_of_pe;            // index into `transports` of the first transport that reaches each PE (-1: none)
  std::unique_ptr<SymmetricHeap> heap;
  bshmemi_state_t dstate{};
  bshmemi_status_t* status_host = nullptr;   // pinned + mapped (GPU) or plain (host mode)
  bshmemi_team_t* team_pool_dev = nullptr;   // device (or host-mode) array [max_teams]
  std::vector<bshmemi_team_t> team_pool_host;
  uint64_t* epochs_dev = nullptr;            // [max_teams][2*BSHMEM_SYNC_SLOTS]
  char* team_area = nullptr;                 // symmetric: per-team sync + LL + scratch
  size_t team_area_bytes = 0, sync_bytes = 0, ll_bytes = 0, scratch_bytes = 0, ll128_bytes = 0;
  std::vector<std::unique_ptr<Team>> teams;  // index = team handle
  std::vector<uint64_t> team_bitmap;         // 1 = free
  int max_teams = 128;
  std::vector<std::pair<StateAddrGetter, std::string>> modules;
  std::atomic<bool> modules_pending{false};  // a module registered after the last state push
  std::vector<std::pair<void*, void*>> driver_modules;  // (CUmodule / CUlibrary, device address of its state copy), see nvshmemx_cumodule_init
  cudaStream_t stream = nullptr;             // internal stream of blocking calls
  std::vector<cudaStream_t> peer_streams;    // non-blocking host RMA, indexed by distance % size
  std::vector<bool> peer_stream_used;
  cudaEvent_t ev_a = nullptr, ev_b = nullptr;
  std::thread watchdog;
  std::atomic<bool> watchdog_stop{false};
  std::atomic<uint32_t> reported_errors{0};
  // counters (observability; dumped at finalize with NVSHMEM_DEBUG=INFO)
  std::atomic<uint64_t> n_put{0}, n_get{0}, bytes_put{0}, bytes_get{0}, n_signal{0}, n_coll{0}, n_alloc{0}, n_barrier{0};
  std::map<std::string, uint64_t> algo_counts;
  uint64_t* host_scratch64 = nullptr;        // symmetric uint64[4 + 2*words] for internal reductions (team index agreement)
  void* malloc_sentinel = nullptr;
  std::atomic<size_t> ce_min_bytes{0};       // copy-engine collectives from this size on (0: never)
};

Runtime& rt();

// The status block is written by device code (or, with the host-memory heap, by host code standing in for it) and
// by API calls, and polled by the watchdog thread: host code touches its words through these relaxed atomics.
inline uint32_t status_load(const volatile uint32_t* p) { return __atomic_load_n((const uint32_t*)p, __ATOMIC_RELAXED); }
inline void status_store(volatile uint32_t* p, uint32_t v) { __atomic_store_n((uint32_t*)p, v, __ATOMIC_RELAXED); }
inline void status_or(volatile uint32_t* p, uint32_t v) { __atomic_fetch_or((uint32_t*)p, v, __ATOMIC_RELAXED); }

// ---- init / finalize (init.cpp)
int runtime_init(const bshmem_uniqueid_t* id, int rank, int nranks, int device_hint, bool hostlib_only, int boot_mode);
int runtime_finalize();
int push_device_state();   // copies dstate into every registered module
void push_pending_modules(); // the same, only if a module registered since the last push
bool is_initialized();
int probe_topology(Runtime& r);
void watchdog_start(Runtime& r);
void watchdog_stop(Runtime& r);

// ---- teams (team.cpp)
int teams_init(Runtime& r);
void teams_finalize(Runtime& r);
void teams_refresh_nvls(Runtime& r);  // after the heap's multicast window changed
void teams_drop_windows(Runtime& r);  // after the heap grew: team windows cover the old size only and are given up
Team* team_get(int handle);
int team_translate_pe(int src_team, int src_pe, int dst_team);
int team_split_strided(int parent, int start, int stride, int size, uint64_t uniqueid, int num_contexts, int* new_team);
int team_split_2d(int parent, int xrange, int* xteam, int* yteam);
int team_create_from_members(int parent, const std::vector<int>& world_members, uint64_t uniqueid, int* new_team);
int team_destroy(int handle);
void team_sync_ptrs(const Runtime& r, int idx, uint64_t* sync, uint64_t* ll, uint64_t* scratch, uint64_t* ll128 = nullptr);

// ---- barriers used by the host paths (coll_host.cu / host_emul.cpp)
int host_barrier_team(int team, cudaStream_t stream, bool blocking);  // quiet + device barrier kernel (GPU) or CPU flags (host mode)
int host_sync_team(int team, cudaStream_t stream, bool blocking);
int host_barrier_all_blocking();
// CPU implementations over the host-memory heap (host_emul.cpp)
int emul_team_sync(int team);
int emul_allreduce_and_u64(int team, uint64_t* data, int words);
// CPU versions of the data collectives (host_emul_coll.cpp); dtype / op as in the device code
int emul_reduce(int team, void* dst, const void* src, size_t n, int dtype, int op);
int emul_reducescatter(int team, void* dst, const void* src, size_t nreduce, int dtype, int op);
int emul_fcollect(int team, void* dst, const void* src, size_t block_bytes);
int emul_alltoall(int team, void* dst, const void* src, size_t block_bytes);
int emul_broadcast(int team, void* dst, const void* src, size_t bytes, int root);

}  // namespace bshmem

extern "C" {
// Called by each CUDA module that carries a copy of the device state (static
// initialiser in the device headers).  Safe before and after initialisation.
void bshmemi_register_module(void* (*getter)(), const char* name);
}
