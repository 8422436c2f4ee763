// Environment-variable option table for the host library.
//
// Every tunable is one row of BSHMEM_OPTIONS below: NAME, kind, default,
// category, help text.  The table is expanded three times: into the fields of
// `Options` (value + `<name>_set` bit), into the parser, and into the listing
// printed by the `nvshmem-info` tool.  Variable names keep the `NVSHMEM_`
// prefix so that job scripts written for NVSHMEM keep working
// (reference: src/include/host/env/env_defs.h, src/host/util/env_vars.cpp).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace bshmem {

enum class OptKind { Bool, Long, Size, Str };
enum class OptCat { OpenShmem, Bootstrap, Collectives, Memory, Transport, Debug, Accepted, Hidden };

// clang-format off
// X(name, ctype, kind, default, category, help)
#define BSHMEM_OPTIONS(X)                                                                                   \
  X(VERSION,               bool,        Bool, false,            OpenShmem,   "Print the library version at start-up")                      \
  X(INFO,                  bool,        Bool, false,            OpenShmem,   "Print every option and its value at start-up")              \
  X(INFO_HIDDEN,           bool,        Bool, false,            Hidden,      "Also print hidden options at start-up")                     \
  X(SYMMETRIC_SIZE,        size_t,      Size, (size_t)1 << 30,  OpenShmem,   "Initial size of the symmetric heap per PE (k/m/g/t suffixes)") \
  X(DEBUG,                 std::string, Str,  "",               OpenShmem,   "Log level: VERSION, WARN, INFO, ABORT or TRACE")            \
  X(DEBUG_SUBSYS,          std::string, Str,  "",               Debug,       "Comma list of subsystems to log: INIT,COLL,P2P,PROXY,TRANSPORT,MEM,BOOTSTRAP,TOPO,UTIL,TEAM,ALL; prefix ^ to invert") \
  X(DEBUG_FILE,            std::string, Str,  "",               Debug,       "Log file name; %h expands to the host name and %p to the pid") \
  X(ENABLE_ERROR_CHECKS,   bool,        Bool, false,            Debug,       "Check symmetry of collective allocation calls")             \
  X(NVTX,                  std::string, Str,  "off",            Debug,       "Comma list of NVTX range groups (off, common, all, init, alloc, launch, coll, wait, memorder, rma, atomic)") \
  X(BOOTSTRAP,             std::string, Str,  "UID",            Bootstrap,   "Bootstrap used by nvshmem_init: UID, PMI, MPI, SHMEM or PLUGIN")             \
  X(BOOTSTRAP_PMI,         std::string, Str,  "PMI",            Bootstrap,   "PMI flavour spoken with the process manager: PMI (PMI-1) or PMI-2") \
  X(BOOTSTRAP_PLUGIN,      std::string, Str,  "",               Bootstrap,   "Path of a bootstrap plugin shared object")                  \
  X(BOOTSTRAP_MPI_PLUGIN,  std::string, Str,  "libbshmem_bootstrap_mpi.so", Bootstrap, "MPI bootstrap plugin: a path, or a file name beside the host library (the plugin opens the job's MPI library itself: NVSHMEM_BOOTSTRAP_MPI_LIB)") \
  X(BOOTSTRAP_SHMEM_PLUGIN, std::string, Str, "libbshmem_bootstrap_shmem.so", Bootstrap, "OpenSHMEM bootstrap plugin: a path, or a file name beside the host library (the plugin finds the OpenSHMEM library itself: NVSHMEM_BOOTSTRAP_SHMEM_LIB; NVSHMEM_BOOTSTRAP_SHMEM_INIT=1 lets it call shmem_init)") \
  X(BOOTSTRAP_UID_SOCK_IFNAME, std::string, Str, "",            Bootstrap,   "Network interface for the UID bootstrap (prefix match; ^ excludes, = exact)") \
  X(BOOTSTRAP_UID_SOCK_FAMILY, std::string, Str, "AF_INET",     Bootstrap,   "Address family for the UID bootstrap: AF_INET or AF_INET6")  \
  X(BOOTSTRAP_UID_SESSION_ID,  std::string, Str, "",            Bootstrap,   "Fixed <address>:<port> of the UID root, replacing the unique-id exchange") \
  X(BOOTSTRAP_TIMEOUT_MS,  long,        Long, 60000,            Bootstrap,   "Milliseconds a bootstrap socket operation may block before it fails") \
  X(DISABLE_NVLS,          bool,        Bool, false,            OpenShmem,   "Do not create NVLink multicast objects even where supported") \
  X(NVLS_TEAM_WINDOWS,     long,        Long, 16,               OpenShmem,   "NVLink multicast windows a PE may hold for teams that do not span the world (0: such teams never get one)") \
  X(DISABLE_CUDA_VMM,      bool,        Bool, false,            Memory,      "Refused on a GPU: the GPU heap needs CUDA virtual memory management (the cudaMalloc + IPC heap of the reference is not built); see NVSHMEM_HEAP_BACKEND") \
  X(REMOTE_TRANSPORT,      std::string, Str,  "none",           Transport,   "Name of a transport plugin (libbshmem_transport_<name>.so) to load beside the built-in load/store transport; none is shipped") \
  X(DISABLE_P2P,           bool,        Bool, false,            Hidden,      "Treat peers as not load/store reachable (init then fails: no remote transport is built)") \
  X(TEST_FAKE_GPU,         long,        Long, -1,               Hidden,      "Host-memory heap only: this PE reports GPU <n> of its host as its device (tests of the same-GPU teams and of the several-PEs-per-GPU status)") \
  X(DISABLE_CE_COLLECTIVES,bool,        Bool, false,            Collectives, "Never use copy engines for on-stream alltoall/fcollect/broadcast") \
  X(CE_COLLECTIVES_MIN_BYTES, size_t,   Size, 0,                Collectives, "On-stream alltoall/fcollect/broadcast of at least this many bytes go through copy engines (0: never)") \
  X(MAX_TEAMS,             long,        Long, 128,              OpenShmem,   "Maximum number of simultaneous teams")                     \
  X(MAX_MEMORY_PER_GPU,    size_t,      Size, (size_t)256 << 30,Memory,      "Virtual address window reserved per PE for the symmetric heap") \
  X(CUMEM_GRANULARITY,     size_t,      Size, (size_t)512 << 20,Memory,      "Granularity of physical heap growth")                      \
  X(CUMEM_HANDLE_TYPE,     std::string, Str,  "FILE_DESCRIPTOR",Memory,      "Shareable handle type for heap chunks: FILE_DESCRIPTOR")    \
  X(HEAP_BACKEND,          std::string, Str,  "AUTO",           Memory,      "AUTO, VMM (GPU memory) or HOST (process-shared host memory, needs no GPU)") \
  X(MAX_CTAS,              long,        Long, 0,                Collectives, "CTAs used by multi-CTA on-stream collectives (0: chosen per collective)") \
  X(SYNC_GPU_SCOPE_RELEASE,bool,        Bool, false,            Collectives, "Team sync releases with a GPU-scope fence instead of a system-scope one (faster by a link round trip when puts are in flight; outside the PTX memory model for cross-GPU observers)") \
  X(BARRIER_DISSEM_KVAL,   long,        Long, 2,                Collectives, "Radix of the dissemination barrier for thread and warp scope") \
  X(BARRIER_TG_DISSEM_KVAL,long,        Long, 2,                Collectives, "Radix of the dissemination barrier for block scope when peers are not all load/store reachable") \
  X(REDUCE_ALGO,           long,        Long, 0,                Collectives, "Force an allreduce algorithm: 0 auto, 1 one-shot pull, 2 two-shot, 3 NVLS one-shot, 4 NVLS two-shot, 5 LL one-shot push") \
  X(REDUCE_NVLS_THRESHOLD, size_t,      Size, 2048,             Collectives, "Element count up to which the NVLS one-shot allreduce is used") \
  X(REDUCE_ONESHOT_THRESHOLD, size_t,   Size, (size_t)256 << 10,Collectives, "Bytes up to which the one-shot allreduce is used when NVLS is absent") \
  X(REDUCE_SCRATCH_SIZE,   size_t,      Size, (size_t)512 << 10, Collectives, "Bytes of per-team scratch for push-based reductions")      \
  X(REDUCE_NTHREADS,       long,        Long, 512,              Collectives, "Threads per CTA for on-stream reductions")                 \
  X(FCOLLECT_ALGO,         long,        Long, 0,                Collectives, "Force an fcollect algorithm: 0 auto, 1 one-shot push, 2 LL, 3 NVLS push") \
  X(LL128_THRESHOLD,       size_t,      Size, 32768,            Collectives, "Bytes per PE up to which fcollect, allreduce and broadcast use 128-byte flag-in-data packets (0: never)") \
  X(FCOLLECT_LL_THRESHOLD, size_t,      Size, 2048,             Collectives, "Bytes up to which fcollect uses the flag-in-data protocol")  \
  X(FCOLLECT_NVLS_THRESHOLD, size_t,    Size, (size_t)16 << 20, Collectives, "Bytes up to which fcollect uses multicast stores when available") \
  X(FCOLLECT_NTHREADS,     long,        Long, 512,              Collectives, "Threads per CTA for on-stream fcollect")                   \
  X(REDUCESCATTER_ALGO,    long,        Long, 0,                Collectives, "Force a reducescatter algorithm: 0 auto, 1 pull, 2 NVLS")  \
  X(REDUCESCATTER_NVLS_THRESHOLD, size_t, Size, (size_t)16 << 20, Collectives, "Bytes up to which the single-CTA NVLS reducescatter is used") \
  X(REDUCESCATTER_NTHREADS,long,        Long, 512,              Collectives, "Threads per CTA for on-stream reducescatter")              \
  X(BCAST_ALGO,            long,        Long, 0,                Collectives, "Force a broadcast algorithm: 0 auto, 1 root push, 2 LL push, 3 NVLS push, 4 pull") \
  X(BCAST_TREE_KVAL,       long,        Long, 2,                Collectives, "Radix of the broadcast tree when peers are not all load/store reachable") \
  X(WAIT_TIMEOUT_MS,       long,        Long, 30000,            Debug,       "Milliseconds a device-side wait may spin before it records a timeout and returns") \
  X(DISABLE_WATCHDOG,      bool,        Bool, false,            Hidden,      "Do not start the host thread that services device-side global_exit and time-outs") \
  X(WATCHDOG_ABORT,        bool,        Bool, false,            Debug,       "Let the watchdog end the process when a device wait times out (default: report only)") \
  X(DEBUG_ATTACH_DELAY,    long,        Long, 0,                Debug,       "Seconds every PE sleeps at the start of initialisation (prints its pid first) so that a debugger can attach") \
  X(CUDA_LIMIT_STACK_SIZE, size_t,      Size, 0,                Debug,       "Per-thread stack size of GPU threads set at initialisation (cudaLimitStackSize); 0 leaves the CUDA default") \
  X(MAX_PEER_STREAMS,      long,        Long, 8,                Transport,   "Internal streams for non-blocking host-initiated copies to different peers (at most one per PE)") \
  X(IGNORE_CUDA_MPS_ACTIVE_THREAD_PERCENTAGE, bool, Bool, false, OpenShmem,  "Several PEs on one GPU under an MPS server: report NVSHMEM_STATUS_FULL_MPG even when their shares of the SMs exceed 100%") \
  X(FCOLLECT_LL128_THRESHOLD, size_t,   Size, 0,                Collectives, "The reference's name for the LL128 limit of fcollect: when set it replaces NVSHMEM_LL128_THRESHOLD (one limit serves fcollect, allreduce and broadcast here)") \
  X(HEAP_KIND,             std::string, Str,  "VIDMEM",         Memory,      "VIDMEM (GPU memory).  SYSMEM (a heap in pinned host memory) is not built and is refused") \
  X(ENABLE_ALIGNED_MALLOC, bool,        Bool, false,            Accepted,    "No effect: every symmetric allocation is already aligned to 512 bytes")   \
  X(REDUCE_RECEXCH_KVAL,   long,        Long, 2,                Accepted,    "No effect: the recursive-exchange all-reduce always pairs PEs (radix 2)") \
  X(REDMAXLOC_ALGO,        long,        Long, 0,                Accepted,    "No effect: the max-location reduction has one algorithm")           \
  X(ASSERT_ATOMICS_SYNC,   bool,        Bool, false,            Accepted,    "No effect: atomics to load/store peers need no proxy synchronisation") \
  X(BOOTSTRAP_TWO_STAGE,   bool,        Bool, false,            Accepted,    "No effect: the bootstraps here are single stage")                   \
  X(BYPASS_ACCESSIBILITY_CHECK, bool,   Bool, false,            Accepted,    "No effect: symmetric-address checks are governed by NVSHMEM_ENABLE_ERROR_CHECKS") \
  X(BYPASS_FLUSH,          bool,        Bool, false,            Accepted,    "No effect: no network transport, nothing to flush")                 \
  X(CUDA_PATH,             std::string, Str,  "",               Accepted,    "No effect: the CUDA driver is found through the dynamic loader")    \
  X(DISABLE_LOCAL_ONLY_PROXY, bool,     Bool, false,            Accepted,    "No effect: there is no proxy thread (a watchdog serves global exit and time-outs)") \
  X(DISABLE_MNNVL,         bool,        Bool, false,            Accepted,    "No effect: one node; multi-node NVLink handles are not used")       \
  X(DISABLE_NCCL,          bool,        Bool, false,            Accepted,    "No effect: collectives never go through NCCL")                      \
  X(DISABLE_NVLS_SHARING,  bool,        Bool, false,            Accepted,    "No effect: every team window is its own multicast object")          \
  X(DISABLE_SELF_WRITE_CE_COLL, bool,   Bool, false,            Accepted,    "No effect: copy-engine collectives always copy the PE's own part too") \
  X(ENABLE_NIC_PE_MAPPING, bool,        Bool, false,            Accepted,    "No effect: no network transport")                                   \
  X(ENABLE_RAIL_OPT,       bool,        Bool, false,            Accepted,    "No effect: no network transport")                                   \
  X(IB_ENABLE_IBGDA,       bool,        Bool, false,            Accepted,    "No effect: no network transport")                                   \
  X(PROXY_REQUEST_BATCH_MAX, long,      Long, 32,               Accepted,    "No effect: there is no proxy thread")
// clang-format on

struct Options {
#define X(name, ctype, kind, dflt, cat, help) \
  ctype name;                                 \
  bool name##_set = false;
  BSHMEM_OPTIONS(X)
#undef X
};

struct OptionInfo {
  const char* name;
  OptKind kind;
  OptCat cat;
  const char* help;
  std::string dflt;
  std::string value;
  bool set;
};

// Parses "20m", "3.1M", ".5g", "1024" into bytes.  Returns false on junk.
bool parse_size(const char* text, size_t* out);
bool parse_bool(const char* text, bool* out);

// Reads every NVSHMEM_<NAME> variable.  Returns 0, or the number of variables
// whose value could not be parsed (each is reported in `errors`).
int options_init(Options* opts, std::vector<std::string>* errors = nullptr);
std::vector<OptionInfo> options_describe(const Options& opts);
const Options& options();       // process-wide, parsed on first use
void options_reload();          // re-read the environment (tests)

}  // namespace bshmem
