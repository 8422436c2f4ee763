// CPU versions of the control-path collectives for the host-memory heap (no
// GPU): the same flag layout and epoch protocol as the device code, executed
// with C++ atomics on the process-shared mapping.  They let bootstrap, heap,
// team and host RMA logic run, and be tested, on a machine without a GPU.
#include <string.h>
#include <time.h>

#include <atomic>
#include <thread>

#include "../state/runtime.h"
#include "../util/env.h"
#include "../util/log.h"

namespace bshmem {

static int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

int emul_team_sync(int team) {
  Runtime& r = rt();
  Team* t = team_get(team);
  if (!t || t->my_pe < 0) return ST_INVALID_VALUE;
  if (t->size == 1) return ST_SUCCESS;
  const int slot = BSHMEM_SYNC_SLOTS - 1;
  uint64_t sync, ll, scratch;
  team_sync_ptrs(r, t->idx, &sync, &ll, &scratch);
  uint64_t* epochs = r.epochs_dev + (size_t)t->idx * 2 * BSHMEM_SYNC_SLOTS;
  const uint64_t epoch = ++epochs[slot];
  uint64_t* flags = (uint64_t*)sync + (size_t)slot * t->size;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  for (int i = 0; i < t->size; ++i) {
    if (i == t->my_pe) continue;
    uint64_t* remote = (uint64_t*)r.heap->translate(flags + t->my_pe, t->members[i]);
    __atomic_store_n(remote, epoch, __ATOMIC_RELEASE);
  }
  const int64_t deadline = now_ms() + options().WAIT_TIMEOUT_MS;
  for (int i = 0; i < t->size; ++i) {
    if (i == t->my_pe) continue;
    while (__atomic_load_n(flags + i, __ATOMIC_ACQUIRE) < epoch) {
      if (now_ms() > deadline) {
        ERROR_PRINT("PE %d: team %d sync timed out waiting for member %d", r.mype, team, i);
        status_or(&r.status_host->error_bits, BSHMEM_ERR_WAIT_TIMEOUT);
        return ST_INTERNAL;
      }
      std::this_thread::yield();
    }
  }
  r.n_barrier++;
  return ST_SUCCESS;
}

int emul_allreduce_and_u64(int team, uint64_t* data, int words) {
  Runtime& r = rt();
  Team* t = team_get(team);
  if (!t || t->my_pe < 0 || words > 6) return ST_INVALID_VALUE;
  for (int i = 0; i < t->size; ++i) {
    uint64_t* remote = (uint64_t*)r.heap->translate(r.host_scratch64 + (size_t)r.mype * 8, t->members[i]);
    memcpy(remote, data, sizeof(uint64_t) * words);
  }
  int st = emul_team_sync(team);
  if (st) return st;
  for (int i = 0; i < t->size; ++i) {
    const uint64_t* got = r.host_scratch64 + (size_t)t->members[i] * 8;
    for (int w = 0; w < words; ++w) data[w] &= got[w];
  }
  return emul_team_sync(team);
}

}  // namespace bshmem
