// Bootstrap over MPI, as a plugin of the host library (NVSHMEM_BOOTSTRAP=MPI, or nvshmemx_init_attr with
// NVSHMEMX_INIT_WITH_MPI_COMM and a pointer to the communicator).
//
// The plugin is not compiled against an MPI installation: it opens the MPI library of the running job at run time
// (the one already in the process, else NVSHMEM_BOOTSTRAP_MPI_LIB, else the usual names) and speaks to it through
// the two binary interfaces in use:
//   * MPICH family (MPICH, Intel MPI, MVAPICH, Cray MPICH): handles are 32-bit integers with fixed values for the
//     predefined objects (MPI_COMM_WORLD = 0x44000000, MPI_BYTE = 0x4c00010d);
//   * Open MPI: handles are pointers to objects that the library exports (ompi_mpi_comm_world, ompi_mpi_byte).
// Which one it is shows in the library's symbols.  Only blocking byte collectives on one duplicated communicator are
// used: MPI_Allgather, MPI_Alltoall, MPI_Barrier.  MPI is initialised here only if the program has not done so, and
// finalised here only in that case.
// (reference: src/modules/bootstrap/mpi/bootstrap_mpi.c, which is compiled against mpi.h)
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../bootstrap/bootstrap.h"

namespace {

enum Abi { ABI_MPICH, ABI_OMPI };

struct MpiLib {
  void* dl = nullptr;
  Abi abi = ABI_MPICH;
  // Entry points, called through casts to the prototype of the detected interface.
  void *Init, *Initialized, *Finalize, *Finalized, *Comm_dup, *Comm_free, *Comm_rank, *Comm_size, *Allgather, *Alltoall, *Barrier, *Abort;
  void *ompi_world = nullptr, *ompi_byte = nullptr;
};

struct MpiState {
  MpiLib lib;
  uintptr_t comm = 0;  // the duplicated communicator: an int (MPICH family) or a pointer (Open MPI), widened
  bool we_initialised = false;
};

constexpr int MPICH_COMM_WORLD = 0x44000000;
constexpr int MPICH_BYTE = 0x4c00010d;

void* sym(void* dl, const char* name) { return dlsym(dl ? dl : RTLD_DEFAULT, name); }

bool open_mpi_library(MpiLib* m) {
  void* dl = nullptr;
  if (!dlsym(RTLD_DEFAULT, "MPI_Allgather")) {  // not in the process yet: open it
    const char* named = getenv("NVSHMEM_BOOTSTRAP_MPI_LIB");
    const char* names[] = {named, "libmpi.so", "libmpi.so.40", "libmpi.so.12", "libmpi_cray.so", "libmpich.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      dl = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (dl) break;
      if (n == named) fprintf(stderr, "mpi bootstrap: cannot open NVSHMEM_BOOTSTRAP_MPI_LIB=%s: %s\n", n, dlerror());
    }
    if (!dl) {
      fprintf(stderr, "mpi bootstrap: no MPI library in the process and none of libmpi.so / libmpi.so.40 / libmpi.so.12 / libmpich.so can be opened "
                      "(set NVSHMEM_BOOTSTRAP_MPI_LIB)\n");
      return false;
    }
  }
  m->dl = dl;
  struct { void** slot; const char* name; } table[] = {
      {&m->Init, "MPI_Init"}, {&m->Initialized, "MPI_Initialized"}, {&m->Finalize, "MPI_Finalize"}, {&m->Finalized, "MPI_Finalized"},
      {&m->Comm_dup, "MPI_Comm_dup"}, {&m->Comm_free, "MPI_Comm_free"}, {&m->Comm_rank, "MPI_Comm_rank"}, {&m->Comm_size, "MPI_Comm_size"},
      {&m->Allgather, "MPI_Allgather"}, {&m->Alltoall, "MPI_Alltoall"}, {&m->Barrier, "MPI_Barrier"}, {&m->Abort, "MPI_Abort"}};
  for (auto& e : table) {
    *e.slot = sym(dl, e.name);
    if (!*e.slot) {
      fprintf(stderr, "mpi bootstrap: the MPI library has no %s\n", e.name);
      return false;
    }
  }
  m->ompi_world = sym(dl, "ompi_mpi_comm_world");
  m->ompi_byte = sym(dl, "ompi_mpi_byte");
  m->abi = (m->ompi_world && m->ompi_byte) ? ABI_OMPI : ABI_MPICH;
  return true;
}

// One set of calls per handle representation.  H is int (MPICH family) or void* (Open MPI).
template <class H>
struct Calls {
  typedef int (*init_fn)(int*, char***);
  typedef int (*flag_fn)(int*);
  typedef int (*void_fn)(void);
  typedef int (*dup_fn)(H, H*);
  typedef int (*free_fn)(H*);
  typedef int (*query_fn)(H, int*);
  typedef int (*coll_fn)(const void*, int, H, void*, int, H, H);
  typedef int (*barrier_fn)(H);
  typedef int (*abort_fn)(H, int);
  static H to_h(uintptr_t v) {
    H h;
    memcpy(&h, &v, sizeof(H));  // little-endian: the low bytes hold a 32-bit handle
    return h;
  }
  static uintptr_t from_h(H h) {
    uintptr_t v = 0;
    memcpy(&v, &h, sizeof(H));
    return v;
  }
};

template <class H>
int start(MpiState* s, H world, H /*byte*/, void* user_comm) {
  typedef Calls<H> C;
  int flag = 0;
  if (((typename C::flag_fn)s->lib.Initialized)(&flag) != 0) return 1;
  if (!flag) {
    if (((typename C::init_fn)s->lib.Init)(nullptr, nullptr) != 0) return 1;
    s->we_initialised = true;
  }
  H parent = world;
  if (user_comm) memcpy(&parent, user_comm, sizeof(H));  // the attribute points at an MPI_Comm
  H dup;
  if (((typename C::dup_fn)s->lib.Comm_dup)(parent, &dup) != 0) return 1;
  s->comm = C::from_h(dup);
  return 0;
}

template <class H>
int rank_size(MpiState* s, int* rank, int* size) {
  typedef Calls<H> C;
  const H comm = C::to_h(s->comm);
  return ((typename C::query_fn)s->lib.Comm_rank)(comm, rank) != 0 || ((typename C::query_fn)s->lib.Comm_size)(comm, size) != 0;
}

template <class H>
H byte_type(const MpiState* s) {
  return sizeof(H) == sizeof(int) ? Calls<H>::to_h((uintptr_t)(unsigned)MPICH_BYTE) : Calls<H>::to_h((uintptr_t)s->lib.ompi_byte);
}

template <class H>
int collective(MpiState* s, void* fn, const void* in, void* out, int bytes) {
  typedef Calls<H> C;
  const H byte = byte_type<H>(s), comm = C::to_h(s->comm);
  return ((typename C::coll_fn)fn)(in, bytes, byte, out, bytes, byte, comm) != 0;
}

template <class H>
int stop(MpiState* s) {
  typedef Calls<H> C;
  int rc = 0, finalized = 0;
  ((typename C::flag_fn)s->lib.Finalized)(&finalized);
  if (!finalized) {
    H comm = C::to_h(s->comm);
    rc |= ((typename C::free_fn)s->lib.Comm_free)(&comm) != 0;
    if (s->we_initialised) rc |= ((typename C::void_fn)s->lib.Finalize)() != 0;
  }
  return rc;
}

#define DISPATCH(s, call_int, call_ptr) ((s)->lib.abi == ABI_MPICH ? (call_int) : (call_ptr))

int mpi_allgather(const void* in, void* out, int bytes, bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  return DISPATCH(s, collective<int>(s, s->lib.Allgather, in, out, bytes), collective<void*>(s, s->lib.Allgather, in, out, bytes));
}
int mpi_alltoall(const void* in, void* out, int bytes, bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  return DISPATCH(s, collective<int>(s, s->lib.Alltoall, in, out, bytes), collective<void*>(s, s->lib.Alltoall, in, out, bytes));
}
int mpi_barrier(bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  if (s->lib.abi == ABI_MPICH) return ((Calls<int>::barrier_fn)s->lib.Barrier)(Calls<int>::to_h(s->comm)) != 0;
  return ((Calls<void*>::barrier_fn)s->lib.Barrier)(Calls<void*>::to_h(s->comm)) != 0;
}
void mpi_global_exit(int status, bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  if (s->lib.abi == ABI_MPICH) ((Calls<int>::abort_fn)s->lib.Abort)(Calls<int>::to_h(s->comm), status);
  else ((Calls<void*>::abort_fn)s->lib.Abort)(Calls<void*>::to_h(s->comm), status);
}
int mpi_finalize(bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  if (!s) return 0;
  const int rc = DISPATCH(s, stop<int>(s), stop<void*>(s));
  delete s;
  h->comm_state = nullptr;
  return rc;
}
int mpi_show_info(bshmem_bootstrap_handle_t* h) {
  MpiState* s = (MpiState*)h->comm_state;
  fprintf(stderr, "bootstrap: MPI (%s interface), rank %d of %d%s\n", s->lib.abi == ABI_MPICH ? "MPICH-family" : "Open MPI", h->pg_rank, h->pg_size,
          s->we_initialised ? ", MPI initialised by the bootstrap" : "");
  return 0;
}

}  // namespace

extern "C" int bshmem_bootstrap_plugin_init(void* attr, bshmem_bootstrap_handle_t* handle, int abi_version) {
  if (abi_version != BSHMEM_BOOTSTRAP_ABI_VERSION) return 3;
  MpiState* s = new MpiState;
  if (!open_mpi_library(&s->lib)) {
    delete s;
    return 4;
  }
  int st;
  if (s->lib.abi == ABI_MPICH) st = start<int>(s, MPICH_COMM_WORLD, MPICH_BYTE, attr);
  else st = start<void*>(s, s->lib.ompi_world, s->lib.ompi_byte, attr);
  int rank = 0, size = 0;
  if (!st) st = DISPATCH(s, rank_size<int>(s, &rank, &size), rank_size<void*>(s, &rank, &size));
  if (st || size < 1 || rank < 0 || rank >= size) {
    fprintf(stderr, "mpi bootstrap: MPI initialisation or communicator duplication failed\n");
    delete s;
    return 5;
  }
  handle->version = BSHMEM_BOOTSTRAP_ABI_VERSION;
  handle->pg_rank = rank;
  handle->pg_size = size;
  handle->allgather = mpi_allgather;
  handle->alltoall = mpi_alltoall;
  handle->barrier = mpi_barrier;
  handle->global_exit = mpi_global_exit;
  handle->finalize = mpi_finalize;
  handle->show_info = mpi_show_info;
  handle->comm_state = s;
  return 0;
}
