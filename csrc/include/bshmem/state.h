// Plain-data state shared between the host library and device code.
//
// The host fills one `bshmemi_state_t` and copies it into the `__constant__`
// instance of every CUDA module that registered itself.  Address translation
// needs no table: the heaps of all PEs are mapped into ONE virtual-address
// reservation as equally sized windows, window k belonging to PE k (the local
// heap is simply window `mype`), so the address of a symmetric object on PE
// `pe` is `ptr + (pe - mype) * heap_stride`.  That holds on an NVSwitch box,
// where every peer is load/store reachable
// (reference: src/include/device_host/nvshmem_types.h, nvshmemi_device_host_state_t).
#pragma once
#include <stdint.h>

#define BSHMEM_MAJOR 3
#define BSHMEM_MINOR 5
#define BSHMEM_PATCH 1
#define BSHMEM_VENDOR_STRING "bshmem (B200-native NVSHMEM-compatible library)"

#define BSHMEM_MAX_PES 128          /* upper bound used for stack arrays in device code */
#define BSHMEM_SYNC_SLOTS 64        /* independent barrier slots per team (one per CTA of a multi-CTA collective) */
#define BSHMEM_TEAM_INVALID (-1)

/* Error bits recorded in the status word by device code (never a trap). */
#define BSHMEM_ERR_WAIT_TIMEOUT 0x1u
#define BSHMEM_ERR_BAD_PE 0x2u
#define BSHMEM_ERR_BAD_ADDRESS 0x4u
#define BSHMEM_ERR_SCRATCH_TOO_SMALL 0x8u
#define BSHMEM_ERR_GLOBAL_EXIT 0x10u
#define BSHMEM_ERR_BAD_TEAM 0x20u

#ifdef __cplusplus
extern "C" {
#endif

/* Block written by device code and polled by the host watchdog thread.  It
 * lives in pinned, mapped host memory. */
typedef struct {
  volatile uint32_t error_bits;      /* OR of BSHMEM_ERR_* */
  volatile uint32_t global_exit_req; /* 1: a kernel called nvshmem_global_exit */
  volatile int32_t global_exit_code;
  volatile uint32_t timeout_count;
  volatile uint64_t timeout_addr;     /* address the first timed-out wait was polling */
  volatile uint64_t timeout_expected; /* value it compared against */
  volatile uint64_t timeout_found;    /* value it last saw */
  volatile uint32_t timeout_where;    /* caller tag (BSHMEM_WHERE_*) */
  volatile uint32_t reserved;
} bshmemi_status_t;

#define BSHMEM_WHERE_WAIT_UNTIL 1
#define BSHMEM_WHERE_SIGNAL_WAIT 2
#define BSHMEM_WHERE_BARRIER 3
#define BSHMEM_WHERE_COLL 4
#define BSHMEM_WHERE_FUSED 5
#define BSHMEM_WHERE_TEAM 6

/* One team as device code sees it.  `pe_of` is null for strided teams. */
typedef struct {
  int32_t my_pe;        /* index of this PE inside the team, -1 if not a member */
  int32_t start;        /* world PE of member 0 */
  int32_t stride;
  int32_t size;
  int32_t team_idx;
  int32_t has_nvls;     /* multicast window bound for exactly this team's members */
  uint64_t mc_base;     /* multicast address of heap offset 0 for this team, or 0 */
  uint64_t sync_base;   /* symmetric: uint64 flags [BSHMEM_SYNC_SLOTS][size] + LL area */
  uint64_t scratch_base;/* symmetric scratch for push-based reductions (2 halves) */
  uint64_t scratch_bytes;
  uint64_t epochs;      /* local device memory: uint64 [BSHMEM_SYNC_SLOTS] barrier epochs + [BSHMEM_SYNC_SLOTS] collective epochs */
  uint64_t pe_of;       /* local device memory: int32 [size] world PE of each member (non-strided teams), else 0 */
  uint64_t ll_base;     /* symmetric flag-in-data buffer (8-byte packets) for small fcollect / allreduce */
  uint64_t ll_bytes;
  uint64_t ll128_base;  /* symmetric area of 128-byte packets: exchange halves, broadcast halves, acknowledgements */
  uint64_t ll128_bytes;
} bshmemi_team_t;

typedef struct {
  int32_t version;
  int32_t mype;
  int32_t npes;
  int32_t mype_node;
  int32_t npes_node;
  int32_t max_teams;
  int32_t job_connectivity;   /* BSHMEM_JOB_* */
  int32_t nvls_world;         /* 1 when TEAM_WORLD has a multicast window */
  uint64_t heap_base;         /* start of this PE's window */
  uint64_t heap_stride;       /* distance between consecutive PEs' windows */
  uint64_t heap_size;         /* bytes of the window that are backed by memory */
  uint64_t mc_base;           /* multicast address of heap offset 0 (TEAM_WORLD) or 0 */
  uint64_t team_pool;         /* device pointer: bshmemi_team_t [max_teams] */
  uint64_t status;            /* device-visible pointer to bshmemi_status_t */
  uint64_t wait_timeout_ns;   /* bound of every device-side spin */
  /* collective tuning, copied from the environment */
  int32_t reduce_algo, fcollect_algo, reducescatter_algo, bcast_algo;
  int32_t barrier_dissem_kval, barrier_tg_dissem_kval, bcast_tree_kval, debug_checks;
  uint64_t reduce_nvls_threshold, reduce_oneshot_threshold;
  uint64_t fcollect_ll_threshold, fcollect_nvls_threshold, reducescatter_nvls_threshold;
  int32_t sync_gpu_release;   /* 1: team sync releases with a GPU-scope fence (NVSHMEM_SYNC_GPU_SCOPE_RELEASE) */
  int32_t reserved0;
  uint64_t ll128_threshold;   /* bytes per PE up to which fcollect / allreduce / broadcast use 128-byte flag-in-data packets */
} bshmemi_state_t;

#define BSHMEM_JOB_GPU_LDST_ATOMICS 0 /* every peer reachable by ld/st/atomics (NVSwitch) */
#define BSHMEM_JOB_GPU_LDST 1
#define BSHMEM_JOB_HOST_ONLY 2        /* host-memory heap: no device code can run */

#ifdef __cplusplus
}
#endif
