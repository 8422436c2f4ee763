#include "bootstrap.h"

#include <dlfcn.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../util/env.h"
#include "../util/log.h"

namespace bshmem {

uint64_t host_hash() {
  char host[1024] = "";
  gethostname(host, sizeof(host) - 1);
  std::string key = host;
  if (const char* extra = getenv("NVSHMEM_HOSTID")) key = extra;  // lets tests fake several nodes
  uint64_t h = 5381;
  for (unsigned char c : key) h = ((h << 5) + h) ^ c;
  return h;
}

int bootstrap_plugin_init(const char* path, void* attr, bshmem_bootstrap_handle_t* handle) {
  std::string p = path ? path : options().BOOTSTRAP_PLUGIN;
  if (p.empty()) {
    ERROR_PRINT("bootstrap: PLUGIN mode needs NVSHMEM_BOOTSTRAP_PLUGIN");
    return BOOT_ERR_PLUGIN;
  }
  void* lib = dlopen(p.c_str(), RTLD_NOW);
  if (!lib) {
    ERROR_PRINT("bootstrap: dlopen(%s) failed: %s", p.c_str(), dlerror());
    return BOOT_ERR_PLUGIN;
  }
  auto fn = (bshmem_bootstrap_plugin_init_fn)dlsym(lib, "bshmem_bootstrap_plugin_init");
  if (!fn) {
    ERROR_PRINT("bootstrap: %s does not export bshmem_bootstrap_plugin_init", p.c_str());
    dlclose(lib);
    return BOOT_ERR_PLUGIN;
  }
  int st = fn(attr, handle, BSHMEM_BOOTSTRAP_ABI_VERSION);
  if (st != 0 || handle->version != BSHMEM_BOOTSTRAP_ABI_VERSION) {
    ERROR_PRINT("bootstrap: plugin %s failed (status %d, ABI %d, expected %d)", p.c_str(), st, handle->version, BSHMEM_BOOTSTRAP_ABI_VERSION);
    return st ? st : BOOT_ERR_VERSION;
  }
  return BOOT_OK;
}

// A plugin that this library ships: `name` is a path, or a bare file name that sits in the directory of this library.
static int shipped_plugin_init(std::string p, void* attr, bshmem_bootstrap_handle_t* handle) {
  if (p.find('/') == std::string::npos) {
    Dl_info info;
    if (dladdr((void*)&shipped_plugin_init, &info) && info.dli_fname) {
      std::string self = info.dli_fname;
      const size_t slash = self.rfind('/');
      if (slash != std::string::npos) p = self.substr(0, slash + 1) + p;
    }
  }
  return bootstrap_plugin_init(p.c_str(), attr, handle);
}
int bootstrap_mpi_init(void* mpi_comm, bshmem_bootstrap_handle_t* handle) { return shipped_plugin_init(options().BOOTSTRAP_MPI_PLUGIN, mpi_comm, handle); }
int bootstrap_shmem_init(bshmem_bootstrap_handle_t* handle) { return shipped_plugin_init(options().BOOTSTRAP_SHMEM_PLUGIN, nullptr, handle); }

int bootstrap_init(int mode, const bshmem_uniqueid_t* id, int rank, int nranks, bshmem_bootstrap_handle_t* handle) {
  memset(handle, 0, sizeof(*handle));
  int st;
  if (mode == BOOT_PLUGIN) st = bootstrap_plugin_init(nullptr, (void*)id, handle);
  else if (mode == BOOT_MPI) st = bootstrap_mpi_init((void*)id, handle);
  else if (mode == BOOT_SHMEM) st = bootstrap_shmem_init(handle);
  else if (mode == BOOT_PMI) st = bootstrap_pmi_init(handle);
  else st = bootstrap_uid_init(id, rank, nranks, handle);
  if (st != BOOT_OK) return st;
  return bootstrap_fill_node_info(handle);
}

int bootstrap_fill_node_info(bshmem_bootstrap_handle_t* h) {
  std::vector<uint64_t> hashes(h->pg_size);
  uint64_t mine = host_hash();
  int st = h->allgather(&mine, hashes.data(), sizeof(uint64_t), h);
  if (st != BOOT_OK) return st;
  int on_node = 0, my_idx = 0;
  for (int r = 0; r < h->pg_size; ++r) {
    if (hashes[r] != mine) continue;
    if (r < h->pg_rank) ++my_idx;
    ++on_node;
  }
  h->mype_node = my_idx;
  h->npes_node = on_node;
  return BOOT_OK;
}

}  // namespace bshmem
