// Out-of-band (CPU) bootstrap seam.  The rest of the host library sees only a
// table of function pointers: allgather, alltoall, barrier, global_exit and
// finalize over `pg_size` processes.  One implementation is built in (UID over
// TCP); another can be loaded from a shared object named by
// NVSHMEM_BOOTSTRAP_PLUGIN that exports `bshmem_bootstrap_plugin_init`
// (reference: src/include/internal/bootstrap_host_transport/nvshmemi_bootstrap_defines.h,
//  src/host/bootstrap/bootstrap.cpp, src/host/bootstrap/bootstrap_loader.cpp).
#pragma once
#include <cstddef>
#include <cstdint>

extern "C" {

#define BSHMEM_BOOTSTRAP_ABI_VERSION 1
#define BSHMEM_UNIQUEID_BYTES 128

typedef struct bshmem_bootstrap_handle {
  int version;
  int pg_rank;
  int pg_size;
  int mype_node;
  int npes_node;
  // Each call returns 0 on success and a non-zero status otherwise; none exits.
  int (*allgather)(const void* sendbuf, void* recvbuf, int bytes_per_rank, struct bshmem_bootstrap_handle* h);
  int (*alltoall)(const void* sendbuf, void* recvbuf, int bytes_per_rank, struct bshmem_bootstrap_handle* h);
  int (*barrier)(struct bshmem_bootstrap_handle* h);
  void (*global_exit)(int status, struct bshmem_bootstrap_handle* h);
  int (*finalize)(struct bshmem_bootstrap_handle* h);
  int (*show_info)(struct bshmem_bootstrap_handle* h);
  void* comm_state;
} bshmem_bootstrap_handle_t;

// Public 128-byte unique id: an int version followed by opaque bytes.
typedef struct {
  int version;
  char internal[BSHMEM_UNIQUEID_BYTES - sizeof(int)];
} bshmem_uniqueid_t;

typedef int (*bshmem_bootstrap_plugin_init_fn)(void* attr, bshmem_bootstrap_handle_t* handle, int abi_version);
}

namespace bshmem {

enum BootstrapMode { BOOT_UID = 0, BOOT_PLUGIN = 1, BOOT_PMI = 2, BOOT_MPI = 3, BOOT_SHMEM = 4 };

enum BootstrapStatus {
  BOOT_OK = 0,
  BOOT_ERR_SOCKET = 1,
  BOOT_ERR_TIMEOUT = 2,
  BOOT_ERR_VERSION = 3,
  BOOT_ERR_ARGS = 4,
  BOOT_ERR_PEER = 5,
  BOOT_ERR_PLUGIN = 6,
};
const char* bootstrap_strerror(int st);

// Rank 0 (or any one process): creates the id and starts the detached root
// thread that collects and redistributes the ranks' listen addresses.
int bootstrap_uid_get_unique_id(bshmem_uniqueid_t* id);
// All ranks: connect through the id.  With NVSHMEM_BOOTSTRAP_UID_SESSION_ID set
// the id may be null: the root address comes from the variable and rank 0
// starts the root thread itself.
int bootstrap_uid_init(const bshmem_uniqueid_t* id, int rank, int nranks, bshmem_bootstrap_handle_t* handle);
// PMI-1 client: rank, size and a socket to the process manager come from PMI_RANK, PMI_SIZE and PMI_FD.
bool bootstrap_pmi_available();
int bootstrap_pmi_init(bshmem_bootstrap_handle_t* handle);
// Loads NVSHMEM_BOOTSTRAP_PLUGIN (or `path`) and calls its init entry point.
int bootstrap_plugin_init(const char* path, void* attr, bshmem_bootstrap_handle_t* handle);
// The MPI bootstrap is a plugin that this library ships (NVSHMEM_BOOTSTRAP_MPI_PLUGIN, looked for beside the host
// library); `mpi_comm` points at the MPI_Comm to duplicate, or is null for MPI_COMM_WORLD.
int bootstrap_mpi_init(void* mpi_comm, bshmem_bootstrap_handle_t* handle);
// The OpenSHMEM bootstrap, shipped the same way (NVSHMEM_BOOTSTRAP_SHMEM_PLUGIN).
int bootstrap_shmem_init(bshmem_bootstrap_handle_t* handle);
// Chooses the mode from NVSHMEM_BOOTSTRAP and initialises `handle`.  With BOOT_PLUGIN and BOOT_MPI `id` carries the
// plugin's attribute (for MPI: the address of the communicator, or null).
int bootstrap_init(int mode, const bshmem_uniqueid_t* id, int rank, int nranks, bshmem_bootstrap_handle_t* handle);
// Fills mype_node / npes_node by all-gathering a hash of the host name.
int bootstrap_fill_node_info(bshmem_bootstrap_handle_t* handle);
uint64_t host_hash();  // DJB2 of the host name (plus NVSHMEM_HOSTID when set)

// Test hook: when non-zero the UID root drops the n-th rank's registration,
// which makes every rank's init end in BOOT_ERR_TIMEOUT (host-side fault injection).
void bootstrap_uid_test_drop_rank(int rank_to_drop);

}  // namespace bshmem
