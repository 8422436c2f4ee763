// C entry points that expose internal pieces (option parser, allocator, raw
// bootstrap) to the Python test-suite.  They are part of the host library so
// that the tests exercise the code that ships, not a copy of it.
#include <string.h>

#include <memory>
#include <vector>

#include "../bootstrap/bootstrap.h"
#include "../heap/allocator.h"
#include "../util/env.h"
#include "../util/log.h"
#include "../util/nvtx.h"

using namespace bshmem;

extern "C" {

int bshmem_test_parse_size(const char* text, unsigned long long* out) {
  size_t v = 0;
  bool ok = parse_size(text, &v);
  if (out) *out = v;
  return ok ? 0 : 1;
}
int bshmem_test_parse_bool(const char* text, int* out) {
  bool v = false;
  bool ok = parse_bool(text, &v);
  if (out) *out = v;
  return ok ? 0 : 1;
}
unsigned bshmem_test_log_subsys(const char* text) { return log_parse_subsys(text ? text : ""); }
unsigned bshmem_test_nvtx_groups(const char* text) { return nvtx_parse(text); }
int bshmem_test_options_count_bad(void) {
  Options o;
  std::vector<std::string> bad;
  return options_init(&o, &bad);
}
// Writes "NAME=value\n" lines for every option into `buf`; returns the length needed.
int bshmem_test_options_dump(char* buf, int cap) {
  Options o;
  options_init(&o);
  std::string s;
  for (auto& i : options_describe(o)) s += std::string(i.name) + "=" + i.value + (i.set ? " (set)" : "") + "\n";
  if (buf && cap > 0) {
    strncpy(buf, s.c_str(), cap - 1);
    buf[cap - 1] = 0;
  }
  return (int)s.size() + 1;
}

// ---- allocator
void* bshmem_test_alloc_new(unsigned long long capacity) {
  auto* a = new HeapAllocator();
  a->add_chunk(0, capacity);
  return a;
}
void bshmem_test_alloc_delete(void* h) { delete (HeapAllocator*)h; }
void bshmem_test_alloc_grow(void* h, unsigned long long offset, unsigned long long size) { ((HeapAllocator*)h)->add_chunk(offset, size); }
long long bshmem_test_alloc_malloc(void* h, unsigned long long size, unsigned long long align) {
  size_t off = 0;
  return ((HeapAllocator*)h)->allocate(size, align, &off) ? (long long)off : -1;
}
int bshmem_test_alloc_free(void* h, unsigned long long offset) { return ((HeapAllocator*)h)->release(offset) ? 0 : 1; }
int bshmem_test_alloc_check(void* h) { return ((HeapAllocator*)h)->check_invariants() ? 0 : 1; }
unsigned long long bshmem_test_alloc_digest(void* h) { return ((HeapAllocator*)h)->history_digest(); }
unsigned long long bshmem_test_alloc_in_use(void* h) { return ((HeapAllocator*)h)->bytes_in_use(); }
unsigned long long bshmem_test_alloc_largest_free(void* h) { return ((HeapAllocator*)h)->largest_free(); }

// ---- raw bootstrap (no heap, no GPU)
void* bshmem_test_boot_init(const bshmem_uniqueid_t* id, int rank, int nranks, int* status) {
  options_reload();
  auto* h = new bshmem_bootstrap_handle_t();
  int st = bootstrap_init(BOOT_UID, id, rank, nranks, h);
  if (status) *status = st;
  if (st != BOOT_OK) {
    delete h;
    return nullptr;
  }
  return h;
}
void* bshmem_test_boot_init_pmi(int* status) {
  options_reload();
  auto* h = new bshmem_bootstrap_handle_t();
  int st = bootstrap_init(BOOT_PMI, nullptr, 0, 0, h);
  if (status) *status = st;
  if (st != BOOT_OK) {
    delete h;
    return nullptr;
  }
  return h;
}
void* bshmem_test_boot_init_plugin(int* status) {
  options_reload();
  auto* h = new bshmem_bootstrap_handle_t();
  int st = bootstrap_init(BOOT_PLUGIN, nullptr, 0, 0, h);
  if (status) *status = st;
  if (st != BOOT_OK) {
    delete h;
    return nullptr;
  }
  return h;
}
int bshmem_test_boot_rank(void* h) { return ((bshmem_bootstrap_handle_t*)h)->pg_rank; }
int bshmem_test_boot_size(void* h) { return ((bshmem_bootstrap_handle_t*)h)->pg_size; }
int bshmem_test_boot_allgather(void* h, const void* send, void* recv, int bytes) {
  auto* b = (bshmem_bootstrap_handle_t*)h;
  return b->allgather(send, recv, bytes, b);
}
int bshmem_test_boot_alltoall(void* h, const void* send, void* recv, int bytes) {
  auto* b = (bshmem_bootstrap_handle_t*)h;
  return b->alltoall(send, recv, bytes, b);
}
int bshmem_test_boot_barrier(void* h) {
  auto* b = (bshmem_bootstrap_handle_t*)h;
  return b->barrier(b);
}
int bshmem_test_boot_node_info(void* h, int* mype_node, int* npes_node) {
  auto* b = (bshmem_bootstrap_handle_t*)h;
  *mype_node = b->mype_node;
  *npes_node = b->npes_node;
  return 0;
}
void bshmem_test_boot_finalize(void* h) {
  auto* b = (bshmem_bootstrap_handle_t*)h;
  b->finalize(b);
  delete b;
}
void bshmem_test_boot_drop_rank(int rank) { bootstrap_uid_test_drop_rank(rank); }
const char* bshmem_test_boot_strerror(int st) { return bootstrap_strerror(st); }
}

// ---- transport seam: capability bits of the built-in load/store transport for a synthetic peer, and the error path
// of the plugin loader (no GPU is touched for peers on another host or on the same device).
#include "../state/runtime.h"
#include "../transport/transport.h"
extern "C" int bshmem_test_transport_caps(int same_host, int same_gpu, unsigned* caps, unsigned* attr) {
  using namespace bshmem;
  bshmem_transport* t = nullptr;
  if (transport_p2p_init(&t) != 0) return 1;
  PeInfo me{}, peer{};
  me.host_hash = 42;
  peer.host_hash = same_host ? 42 : 43;
  memset(me.uuid, 7, 16);
  memset(peer.uuid, same_gpu ? 7 : 9, 16);
  snprintf(peer.pci_bus_id, sizeof(peer.pci_bus_id), "0000:ff:1f.0");
  uint32_t c = 0;
  int st = t->ops.can_reach_peer(t, &me, &peer, 0, &c);
  *caps = c;
  *attr = t->attr;
  transport_destroy(t);
  return st;
}
extern "C" int bshmem_test_transport_load(const char* name) {
  bshmem::bshmem_transport* t = nullptr;
  int st = bshmem::transport_load_plugin(name, &t);
  if (st == 0) bshmem::transport_destroy(t);
  return st;
}
