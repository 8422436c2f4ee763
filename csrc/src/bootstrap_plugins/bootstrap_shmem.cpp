// Bootstrap over an OpenSHMEM library, as a plugin of the host library (NVSHMEM_BOOTSTRAP=SHMEM, or
// nvshmemx_init_attr with NVSHMEMX_INIT_WITH_SHMEM): for programs that already run under an OpenSHMEM launcher
// (oshrun, srun with a SHMEM library) and want this library beside it.
//
// Like the MPI plugin it is not compiled against an installation: it looks the entry points up in the process (or
// opens NVSHMEM_BOOTSTRAP_SHMEM_LIB / liboshmem.so / libsma.so / libshmem.so) and uses only calls whose binary form
// is the same in every implementation: shmem_init, shmem_my_pe, shmem_n_pes, shmem_malloc, shmem_free, shmem_putmem,
// shmem_quiet, shmem_barrier_all, shmem_finalize, shmem_global_exit.  The collective routines of OpenSHMEM are
// avoided on purpose: their work arrays (pSync) have implementation-defined sizes and initial values that only the
// implementation's header knows.
//   allgather: every PE puts its contribution into slot `rank` of a symmetric buffer on every PE, then barrier_all;
//   alltoall:  every PE puts piece p into slot `rank` of PE p's buffer, then barrier_all.
// A second barrier_all after the result has been copied out lets the buffer be reused by the next call.
// Who initialises OpenSHMEM: a library that was already in the process belongs to the program, which has initialised
// it; a library that the plugin had to open itself is initialised (and finalised) by the plugin.
// NVSHMEM_BOOTSTRAP_SHMEM_INIT=1 / 0 overrides that guess.
// (reference: src/modules/bootstrap/shmem/bootstrap_shmem.c, compiled against shmem.h)
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../bootstrap/bootstrap.h"

namespace {

struct ShmemLib {
  void (*init)(void);
  void (*finalize)(void);
  int (*my_pe)(void);
  int (*n_pes)(void);
  void* (*malloc_)(size_t);
  void (*free_)(void*);
  void (*putmem)(void*, const void*, size_t, int);
  void (*quiet)(void);
  void (*barrier_all)(void);
  void (*global_exit)(int);
};

struct ShmemState {
  ShmemLib lib{};
  int rank = 0, size = 1;
  char* buf = nullptr;  // symmetric exchange buffer: `size` slots of `slot_bytes`
  size_t slot_bytes = 0;
  bool we_initialised = false;
};

bool open_shmem_library(ShmemLib* l, bool* opened_here) {
  void* dl = nullptr;
  *opened_here = false;
  if (!dlsym(RTLD_DEFAULT, "shmem_putmem")) {
    const char* named = getenv("NVSHMEM_BOOTSTRAP_SHMEM_LIB");
    const char* names[] = {named, "liboshmem.so", "liboshmem.so.40", "libsma.so", "libshmem.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      dl = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (dl) break;
      if (n == named) fprintf(stderr, "shmem bootstrap: cannot open NVSHMEM_BOOTSTRAP_SHMEM_LIB=%s: %s\n", n, dlerror());
    }
    if (!dl) {
      fprintf(stderr, "shmem bootstrap: no OpenSHMEM library in the process and none of liboshmem.so / libsma.so / libshmem.so can be opened "
                      "(set NVSHMEM_BOOTSTRAP_SHMEM_LIB)\n");
      return false;
    }
    *opened_here = true;
  }
  struct { void** slot; const char* name; } table[] = {
      {(void**)&l->init, "shmem_init"}, {(void**)&l->finalize, "shmem_finalize"}, {(void**)&l->my_pe, "shmem_my_pe"}, {(void**)&l->n_pes, "shmem_n_pes"},
      {(void**)&l->malloc_, "shmem_malloc"}, {(void**)&l->free_, "shmem_free"}, {(void**)&l->putmem, "shmem_putmem"}, {(void**)&l->quiet, "shmem_quiet"},
      {(void**)&l->barrier_all, "shmem_barrier_all"}, {(void**)&l->global_exit, "shmem_global_exit"}};
  for (auto& e : table) {
    *e.slot = dlsym(dl ? dl : RTLD_DEFAULT, e.name);
    if (!*e.slot) {
      fprintf(stderr, "shmem bootstrap: the OpenSHMEM library has no %s\n", e.name);
      return false;
    }
  }
  return true;
}

// Makes the exchange buffer hold `size` slots of at least `bytes`.  Collective: every PE asks for the same size at
// the same call, because the bootstrap's calls are collective with equal arguments.
int ensure(ShmemState* s, size_t bytes) {
  if (bytes <= s->slot_bytes) return 0;
  if (s->buf) s->lib.free_(s->buf);  // shmem_free is collective and ends with a barrier
  size_t want = 4096;
  while (want < bytes) want *= 2;
  s->buf = (char*)s->lib.malloc_(want * (size_t)s->size);
  s->slot_bytes = s->buf ? want : 0;
  return s->buf ? 0 : 1;
}

int boot_allgather(const void* in, void* out, int bytes, bshmem_bootstrap_handle_t* h) {
  ShmemState* s = (ShmemState*)h->comm_state;
  if (bytes < 0 || ensure(s, (size_t)bytes)) return 1;
  for (int o = 0; o < s->size; ++o) {
    const int pe = (s->rank + o) % s->size;
    s->lib.putmem(s->buf + (size_t)s->rank * s->slot_bytes, in, (size_t)bytes, pe);
  }
  s->lib.barrier_all();  // completes the puts of every PE
  for (int r = 0; r < s->size; ++r) memcpy((char*)out + (size_t)r * bytes, s->buf + (size_t)r * s->slot_bytes, (size_t)bytes);
  s->lib.barrier_all();  // everybody has read: the buffer may be written again
  return 0;
}

int boot_alltoall(const void* in, void* out, int bytes, bshmem_bootstrap_handle_t* h) {
  ShmemState* s = (ShmemState*)h->comm_state;
  if (bytes < 0 || ensure(s, (size_t)bytes)) return 1;
  for (int o = 0; o < s->size; ++o) {
    const int pe = (s->rank + o) % s->size;
    s->lib.putmem(s->buf + (size_t)s->rank * s->slot_bytes, (const char*)in + (size_t)pe * bytes, (size_t)bytes, pe);
  }
  s->lib.barrier_all();
  for (int r = 0; r < s->size; ++r) memcpy((char*)out + (size_t)r * bytes, s->buf + (size_t)r * s->slot_bytes, (size_t)bytes);
  s->lib.barrier_all();
  return 0;
}

int boot_barrier(bshmem_bootstrap_handle_t* h) {
  ((ShmemState*)h->comm_state)->lib.barrier_all();
  return 0;
}

void boot_exit(int status, bshmem_bootstrap_handle_t* h) { ((ShmemState*)h->comm_state)->lib.global_exit(status); }

int boot_finalize(bshmem_bootstrap_handle_t* h) {
  ShmemState* s = (ShmemState*)h->comm_state;
  if (!s) return 0;
  if (s->buf) s->lib.free_(s->buf);
  if (s->we_initialised) s->lib.finalize();
  delete s;
  h->comm_state = nullptr;
  return 0;
}

int boot_show(bshmem_bootstrap_handle_t* h) {
  ShmemState* s = (ShmemState*)h->comm_state;
  fprintf(stderr, "bootstrap: OpenSHMEM, PE %d of %d%s\n", s->rank, s->size, s->we_initialised ? ", OpenSHMEM initialised by the bootstrap" : "");
  return 0;
}

}  // namespace

extern "C" int bshmem_bootstrap_plugin_init(void* attr, bshmem_bootstrap_handle_t* handle, int abi_version) {
  (void)attr;
  if (abi_version != BSHMEM_BOOTSTRAP_ABI_VERSION) return 3;
  ShmemState* s = new ShmemState;
  bool opened_here = false;
  if (!open_shmem_library(&s->lib, &opened_here)) {
    delete s;
    return 4;
  }
  const char* do_init = getenv("NVSHMEM_BOOTSTRAP_SHMEM_INIT");
  if (do_init && *do_init ? atoi(do_init) != 0 : opened_here) {
    s->lib.init();
    s->we_initialised = true;
  }
  s->rank = s->lib.my_pe();
  s->size = s->lib.n_pes();
  if (s->size < 1 || s->rank < 0 || s->rank >= s->size) {
    fprintf(stderr, "shmem bootstrap: OpenSHMEM reports PE %d of %d: is it initialised? (NVSHMEM_BOOTSTRAP_SHMEM_INIT=1 makes the bootstrap call shmem_init)\n",
            s->rank, s->size);
    delete s;
    return 5;
  }
  handle->version = BSHMEM_BOOTSTRAP_ABI_VERSION;
  handle->pg_rank = s->rank;
  handle->pg_size = s->size;
  handle->allgather = boot_allgather;
  handle->alltoall = boot_alltoall;
  handle->barrier = boot_barrier;
  handle->global_exit = boot_exit;
  handle->finalize = boot_finalize;
  handle->show_info = boot_show;
  handle->comm_state = s;
  return 0;
}
