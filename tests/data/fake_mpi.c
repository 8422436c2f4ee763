/* A stand-in for an MPI library, for the CPU tests of the MPI bootstrap plugin: the dozen entry points that the
 * plugin uses, over files in a directory (FAKE_MPI_DIR) with rank and size from FAKE_MPI_RANK / FAKE_MPI_SIZE (else RANK / WORLD_SIZE).
 * Built twice: with the MPICH family's binary interface (integer handles with the predefined values) and, with
 * -DFAKE_OMPI, with Open MPI's (handles are pointers to exported objects).  Every call checks the handles it is
 * given, so a plugin that mixes the interfaces up fails loudly. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#ifdef FAKE_OMPI
struct ompi_communicator_t { int id; };
struct ompi_datatype_t { int size; };
struct ompi_communicator_t ompi_mpi_comm_world = {1};
struct ompi_datatype_t ompi_mpi_byte = {1};
typedef struct ompi_communicator_t* MPI_Comm;
typedef struct ompi_datatype_t* MPI_Datatype;
static struct ompi_communicator_t dups[8];
static int comm_ok(MPI_Comm c) { return c == &ompi_mpi_comm_world || (c >= dups && c < dups + 8 && c->id > 1); }
static int byte_ok(MPI_Datatype t) { return t == &ompi_mpi_byte; }
static int comm_id(MPI_Comm c) { return c->id; }
#else
typedef int MPI_Comm;
typedef int MPI_Datatype;
#define WORLD 0x44000000
#define BYTE 0x4c00010d
static int comm_ok(MPI_Comm c) { return c == WORLD || (c > (int)0x84000000 && c <= (int)0x84000008); }
static int byte_ok(MPI_Datatype t) { return t == BYTE; }
static int comm_id(MPI_Comm c) { return c == WORLD ? 1 : c - (int)0x84000000 + 1; }
#endif

static int initialized, finalized, ndups, rank, size;
static unsigned long long seq[16];
static const char* dir;

static void die(const char* what) {
  fprintf(stderr, "fake MPI: %s\n", what);
  abort();
}

int MPI_Initialized(int* flag) { *flag = initialized; return 0; }
int MPI_Finalized(int* flag) { *flag = finalized; return 0; }
int MPI_Init(int* argc, char*** argv) {
  (void)argc; (void)argv;
  dir = getenv("FAKE_MPI_DIR");
  const char* r = getenv("FAKE_MPI_RANK") ? getenv("FAKE_MPI_RANK") : getenv("RANK");
  const char* n = getenv("FAKE_MPI_SIZE") ? getenv("FAKE_MPI_SIZE") : getenv("WORLD_SIZE");
  if (!dir || !r || !n) die("FAKE_MPI_DIR and a rank and size (FAKE_MPI_RANK / FAKE_MPI_SIZE, or RANK / WORLD_SIZE) are not set");
  rank = atoi(r);
  size = atoi(n);
  initialized = 1;
  return 0;
}
int MPI_Finalize(void) {
  if (!initialized || finalized) die("MPI_Finalize out of order");
  finalized = 1;
  char path[512];
  snprintf(path, sizeof path, "%s/finalized.%d", dir, rank);
  FILE* f = fopen(path, "w");
  if (f) fclose(f);
  return 0;
}
int MPI_Comm_dup(MPI_Comm c, MPI_Comm* out) {
  if (!initialized || !comm_ok(c)) die("MPI_Comm_dup: bad communicator handle");
  ++ndups;
#ifdef FAKE_OMPI
  dups[ndups].id = 1 + ndups;
  *out = &dups[ndups];
#else
  *out = (int)0x84000000 + ndups;
#endif
  return 0;
}
int MPI_Comm_free(MPI_Comm* c) {
  if (!comm_ok(*c) || comm_id(*c) == 1) die("MPI_Comm_free: bad communicator handle");
  return 0;
}
int MPI_Comm_rank(MPI_Comm c, int* r) { if (!comm_ok(c)) die("MPI_Comm_rank: bad handle"); *r = rank; return 0; }
int MPI_Comm_size(MPI_Comm c, int* s) { if (!comm_ok(c)) die("MPI_Comm_size: bad handle"); *s = size; return 0; }
int MPI_Abort(MPI_Comm c, int code) { (void)c; _exit(code); }

static void put_file(int comm, unsigned long long n, const void* data, size_t bytes) {
  char tmp[640], path[600];
  snprintf(path, sizeof path, "%s/c%d.%llu.%d", dir, comm, n, rank);
  snprintf(tmp, sizeof tmp, "%s.tmp", path);
  FILE* f = fopen(tmp, "wb");
  if (!f || (bytes && fwrite(data, 1, bytes, f) != bytes) || fclose(f) != 0 || rename(tmp, path) != 0) die("cannot write an exchange file");
}
static void get_file(int comm, unsigned long long n, int from, size_t offset, void* out, size_t bytes) {
  char path[600];
  snprintf(path, sizeof path, "%s/c%d.%llu.%d", dir, comm, n, from);
  for (int tries = 0; tries < 60000; ++tries) {
    FILE* f = fopen(path, "rb");
    if (f) {
      if (fseek(f, (long)offset, SEEK_SET) != 0 || (bytes && fread(out, 1, bytes, f) != bytes)) die("short exchange file");
      fclose(f);
      return;
    }
    struct timespec ts = {0, 1000000};
    nanosleep(&ts, NULL);
  }
  die("a peer did not arrive within a minute");
}

int MPI_Allgather(const void* in, int n_in, MPI_Datatype t_in, void* out, int n_out, MPI_Datatype t_out, MPI_Comm c) {
  if (!comm_ok(c) || !byte_ok(t_in) || !byte_ok(t_out) || n_in != n_out) die("MPI_Allgather: bad handle or count");
  const int id = comm_id(c);
  const unsigned long long n = seq[id]++;
  put_file(id, n, in, (size_t)n_in);
  for (int r = 0; r < size; ++r) get_file(id, n, r, 0, (char*)out + (size_t)r * n_out, (size_t)n_out);
  return 0;
}
int MPI_Alltoall(const void* in, int n_in, MPI_Datatype t_in, void* out, int n_out, MPI_Datatype t_out, MPI_Comm c) {
  if (!comm_ok(c) || !byte_ok(t_in) || !byte_ok(t_out) || n_in != n_out) die("MPI_Alltoall: bad handle or count");
  const int id = comm_id(c);
  const unsigned long long n = seq[id]++;
  put_file(id, n, in, (size_t)n_in * size);
  for (int r = 0; r < size; ++r) get_file(id, n, r, (size_t)rank * n_in, (char*)out + (size_t)r * n_out, (size_t)n_out);
  return 0;
}
int MPI_Barrier(MPI_Comm c) {
  if (!comm_ok(c)) die("MPI_Barrier: bad handle");
  const int id = comm_id(c);
  const unsigned long long n = seq[id]++;
  char none = 0;
  put_file(id, n, &none, 1);
  for (int r = 0; r < size; ++r) get_file(id, n, r, 0, &none, 1);
  return 0;
}
