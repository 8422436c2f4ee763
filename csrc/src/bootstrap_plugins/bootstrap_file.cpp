// A bootstrap plugin: the out-of-band exchange goes through files in a directory that every process can reach
// (a shared file system across nodes, /dev/shm or /tmp on one node).  It shows the plugin seam of the host library
// (NVSHMEM_BOOTSTRAP=PLUGIN, NVSHMEM_BOOTSTRAP_PLUGIN=<this .so>) and serves launchers that can hand a process its
// rank but no socket:
//   BSHMEM_FILE_BOOTSTRAP_DIR   directory for the exchange (must exist; one per job)
//   BSHMEM_FILE_BOOTSTRAP_RANK / _SIZE   this process's rank and the job size (default: RANK / WORLD_SIZE)
// Every collective call has a sequence number; a rank publishes its contribution as <dir>/<seq>.<rank> (written to a
// temporary name and renamed, so readers never see a partial file) and polls for the others' files, with a bound.
// (reference: the plugin architecture of src/modules/bootstrap/* and src/host/bootstrap/bootstrap_loader.cpp)
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../bootstrap/bootstrap.h"

namespace {

struct FileState {
  std::string dir;
  int rank = 0, size = 1;
  unsigned long long seq = 0;
  long timeout_ms = 60000;
};

long long now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (long long)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

std::string name_of(const FileState* s, unsigned long long seq, int rank) { return s->dir + "/" + std::to_string(seq) + "." + std::to_string(rank); }

int publish(const FileState* s, unsigned long long seq, const void* data, size_t bytes) {
  const std::string final_name = name_of(s, seq, s->rank), tmp = final_name + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return 1;
  const bool ok = bytes == 0 || fwrite(data, 1, bytes, f) == bytes;
  if (fclose(f) != 0 || !ok) return 1;
  return rename(tmp.c_str(), final_name.c_str()) == 0 ? 0 : 1;
}

int fetch(const FileState* s, unsigned long long seq, int rank, size_t offset, void* out, size_t bytes) {
  const std::string path = name_of(s, seq, rank);
  const long long deadline = now_ms() + s->timeout_ms;
  for (;;) {
    FILE* f = fopen(path.c_str(), "rb");
    if (f) {
      int rc = 0;
      if (fseek(f, (long)offset, SEEK_SET) != 0 || (bytes && fread(out, 1, bytes, f) != bytes)) rc = 1;
      fclose(f);
      return rc;
    }
    if (now_ms() > deadline) {
      fprintf(stderr, "file bootstrap: rank %d gave up waiting for %s\n", s->rank, path.c_str());
      return 2;  // time-out
    }
    usleep(500);
  }
}

// A rank removes its own file of the previous call once it has read everyone's file of this call: a rank publishes
// call k only after it has finished reading call k-1, so by then nobody needs the older file any more.
void retire(const FileState* s, unsigned long long seq) {
  if (seq >= 1) unlink(name_of(s, seq - 1, s->rank).c_str());
}

bool exists(const std::string& path) {
  struct stat sb;
  return stat(path.c_str(), &sb) == 0;
}
// Polls until `path` exists (want = true) or is gone (want = false); false on time-out.
bool wait_path(const FileState* s, const std::string& path, bool want) {
  const long long deadline = now_ms() + s->timeout_ms;
  while (exists(path) != want) {
    if (now_ms() > deadline) return false;
    usleep(500);
  }
  return true;
}

int file_allgather(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  FileState* s = (FileState*)h->comm_state;
  const unsigned long long seq = s->seq++;
  if (publish(s, seq, sendbuf, (size_t)bytes)) return 1;
  for (int r = 0; r < s->size; ++r) {
    if (r == s->rank) memcpy((char*)recvbuf + (size_t)r * bytes, sendbuf, (size_t)bytes);
    else if (int st = fetch(s, seq, r, 0, (char*)recvbuf + (size_t)r * bytes, (size_t)bytes)) return st;
  }
  retire(s, seq);
  return 0;
}

int file_alltoall(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  FileState* s = (FileState*)h->comm_state;
  const unsigned long long seq = s->seq++;
  if (publish(s, seq, sendbuf, (size_t)bytes * s->size)) return 1;  // my whole send buffer; reader r takes block r
  for (int r = 0; r < s->size; ++r) {
    if (r == s->rank) memcpy((char*)recvbuf + (size_t)r * bytes, (const char*)sendbuf + (size_t)r * bytes, (size_t)bytes);
    else if (int st = fetch(s, seq, r, (size_t)s->rank * bytes, (char*)recvbuf + (size_t)r * bytes, (size_t)bytes)) return st;
  }
  retire(s, seq);
  return 0;
}

int file_barrier(bshmem_bootstrap_handle_t* h) {
  char token = 0;
  std::vector<char> all(((FileState*)h->comm_state)->size);
  return file_allgather(&token, all.data(), 1, h);
}

void file_global_exit(int status, bshmem_bootstrap_handle_t*) { _exit(status); }

// Leaving without leftovers: a file may only be removed when every reader is done with it, so the last round is
// asymmetric.  Every rank but 0 announces itself (fin.<rank>) and waits for rank 0's release; rank 0 publishes the
// release once all have announced, which also means that everyone has finished the last collective; each rank then
// removes its files, and rank 0 removes the release when the announcements are gone.
int file_finalize(bshmem_bootstrap_handle_t* h) {
  FileState* s = (FileState*)h->comm_state;
  if (!s) return 0;
  const std::string release = s->dir + "/fin.release";
  auto fin = [&](int r) { return s->dir + "/fin." + std::to_string(r); };
  auto drop_mine = [&]() {
    if (s->seq >= 1) unlink(name_of(s, s->seq - 1, s->rank).c_str());
  };
  int rc = 0;
  if (s->size > 1) {
    if (s->rank != 0) {
      FILE* f = fopen(fin(s->rank).c_str(), "wb");
      if (f) fclose(f);
      if (!wait_path(s, release, true)) rc = 2;
      drop_mine();
      unlink(fin(s->rank).c_str());
    } else {
      for (int r = 1; r < s->size && !rc; ++r)
        if (!wait_path(s, fin(r), true)) rc = 2;
      FILE* f = fopen(release.c_str(), "wb");
      if (f) fclose(f);
      for (int r = 1; r < s->size; ++r)
        if (!wait_path(s, fin(r), false)) rc = 2;
      unlink(release.c_str());
      drop_mine();
    }
  } else {
    drop_mine();
  }
  delete s;
  h->comm_state = nullptr;
  return rc;
}

int file_show_info(bshmem_bootstrap_handle_t* h) {
  FileState* s = (FileState*)h->comm_state;
  fprintf(stderr, "file bootstrap: rank %d of %d through %s\n", s->rank, s->size, s->dir.c_str());
  return 0;
}

}  // namespace

extern "C" int bshmem_bootstrap_plugin_init(void* attr, bshmem_bootstrap_handle_t* handle, int abi_version) {
  (void)attr;
  if (abi_version != BSHMEM_BOOTSTRAP_ABI_VERSION) return 3;
  const char* dir = getenv("BSHMEM_FILE_BOOTSTRAP_DIR");
  const char* rank = getenv("BSHMEM_FILE_BOOTSTRAP_RANK") ? getenv("BSHMEM_FILE_BOOTSTRAP_RANK") : getenv("RANK");
  const char* size = getenv("BSHMEM_FILE_BOOTSTRAP_SIZE") ? getenv("BSHMEM_FILE_BOOTSTRAP_SIZE") : getenv("WORLD_SIZE");
  struct stat sb;
  if (!dir || !rank || !size || stat(dir, &sb) != 0 || !S_ISDIR(sb.st_mode)) {
    fprintf(stderr, "file bootstrap: set BSHMEM_FILE_BOOTSTRAP_DIR (an existing directory) and a rank and size\n");
    return 4;
  }
  FileState* s = new FileState;
  s->dir = dir;
  s->rank = atoi(rank);
  s->size = atoi(size);
  if (const char* t = getenv("NVSHMEM_BOOTSTRAP_TIMEOUT_MS")) s->timeout_ms = atol(t) > 0 ? atol(t) : s->timeout_ms;
  if (s->size < 1 || s->rank < 0 || s->rank >= s->size) {
    delete s;
    return 4;
  }
  handle->version = BSHMEM_BOOTSTRAP_ABI_VERSION;
  handle->pg_rank = s->rank;
  handle->pg_size = s->size;
  handle->allgather = file_allgather;
  handle->alltoall = file_alltoall;
  handle->barrier = file_barrier;
  handle->global_exit = file_global_exit;
  handle->finalize = file_finalize;
  handle->show_info = file_show_info;
  handle->comm_state = s;
  return 0;
}
