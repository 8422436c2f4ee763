/* A stand-in for an OpenSHMEM library, for the CPU tests of the OpenSHMEM bootstrap plugin: the ten entry points
 * that the plugin uses.  Every PE's symmetric heap is a file in FAKE_SHMEM_DIR mapped shared by all PEs; puts are
 * memcpy into the target's mapping; the barrier is a counter and a generation word in a shared control file.  PE and
 * job size come from FAKE_SHMEM_RANK / FAKE_SHMEM_SIZE (else RANK / WORLD_SIZE). */
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <time.h>
#include <unistd.h>

#define HEAP_BYTES ((size_t)32 << 20)
#define MAX_PES 64

struct ctl { volatile int count; volatile int gen; };
static int pe = -1, npes = 0, initialized;
static char* heap[MAX_PES];
static size_t brk_;
static struct ctl* ctl;
static const char* dir;

static void die(const char* what) {
  fprintf(stderr, "fake OpenSHMEM: %s\n", what);
  abort();
}
static void* map_file(const char* name, size_t bytes) {
  char path[600];
  snprintf(path, sizeof path, "%s/%s", dir, name);
  int fd = open(path, O_RDWR | O_CREAT, 0600);
  if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) die("cannot create a heap file");
  void* p = mmap(NULL, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) die("mmap failed");
  return p;
}

void shmem_barrier_all(void) {
  if (!initialized) die("shmem_barrier_all before shmem_init");
  __sync_synchronize();
  const int g = ctl->gen;
  if (__sync_add_and_fetch(&ctl->count, 1) == npes) {
    ctl->count = 0;
    __sync_synchronize();
    ctl->gen = g + 1;
  } else {
    for (long spins = 0; ctl->gen == g; ++spins) {
      if (spins > 60000) die("a PE did not reach the barrier within a minute");
      struct timespec ts = {0, 1000000};
      nanosleep(&ts, NULL);
    }
  }
  __sync_synchronize();
}
void shmem_init(void) {
  if (initialized) die("shmem_init twice");
  dir = getenv("FAKE_SHMEM_DIR");
  const char* r = getenv("FAKE_SHMEM_RANK") ? getenv("FAKE_SHMEM_RANK") : getenv("RANK");
  const char* n = getenv("FAKE_SHMEM_SIZE") ? getenv("FAKE_SHMEM_SIZE") : getenv("WORLD_SIZE");
  if (!dir || !r || !n) die("FAKE_SHMEM_DIR and a rank and size are not set");
  pe = atoi(r);
  npes = atoi(n);
  if (npes < 1 || npes > MAX_PES || pe < 0 || pe >= npes) die("bad rank or size");
  ctl = (struct ctl*)map_file("ctl", 4096);
  for (int p = 0; p < npes; ++p) {  // every PE creates (or finds) every file: ftruncate to the same size is harmless
    char name[32];
    snprintf(name, sizeof name, "heap.%d", p);
    heap[p] = (char*)map_file(name, HEAP_BYTES);
  }
  initialized = 1;
  shmem_barrier_all();
}
void shmem_finalize(void) {
  if (!initialized) die("shmem_finalize before shmem_init");
  shmem_barrier_all();
  char path[600];
  snprintf(path, sizeof path, "%s/finalized.%d", dir, pe);
  FILE* f = fopen(path, "w");
  if (f) fclose(f);
  initialized = 0;
}
int shmem_my_pe(void) { return initialized ? pe : -1; }
int shmem_n_pes(void) { return initialized ? npes : 0; }
void* shmem_malloc(size_t bytes) {
  if (!initialized) die("shmem_malloc before shmem_init");
  bytes = (bytes + 63) & ~(size_t)63;
  if (brk_ + bytes > HEAP_BYTES) return NULL;
  void* p = heap[pe] + brk_;
  brk_ += bytes;
  shmem_barrier_all();
  return p;
}
void shmem_free(void* p) {
  (void)p;  /* a bump allocator: nothing comes back */
  shmem_barrier_all();
}
void shmem_putmem(void* dst, const void* src, size_t bytes, int target) {
  if (!initialized || target < 0 || target >= npes) die("shmem_putmem: bad target PE");
  const size_t off = (size_t)((char*)dst - heap[pe]);
  if (off > HEAP_BYTES || off + bytes > HEAP_BYTES) die("shmem_putmem: destination is not symmetric");
  memcpy(heap[target] + off, src, bytes);
}
void shmem_quiet(void) { __sync_synchronize(); }
void shmem_global_exit(int status) { _exit(status); }
