// Teams: the predefined ones, strided and 2-D splits, unique-id teams built
// from arbitrary PE sets, PE translation and destruction.
//
// Every team owns slot `idx` of a per-PE *team area* in the symmetric heap,
// reserved once at start-up for NVSHMEM_MAX_TEAMS teams (creating a team must
// not allocate: only the parent's members take part, and an allocation by a
// subset of PEs would break the symmetry of the heap).  A slot holds
//   [ sync flags: BSHMEM_SYNC_SLOTS x npes uint64 ][ flag-in-data buffer ][ scratch, two halves ]
// so a multi-CTA collective gives each CTA its own row of barrier flags rather
// than cloning the team.  Barrier flags carry ever-increasing epochs and are
// cleared when the team is destroyed.  The team index is agreed by AND-ing the
// members' free-slot bitmaps
// (reference behaviour: src/host/team/team_internal.cpp, team.cu).
#include <string.h>

#include <algorithm>
#include <chrono>
#include <thread>

#include "../state/runtime.h"
#include "../util/env.h"
#include "../util/log.h"

namespace bshmem {

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

enum { TEAM_WORLD = 0, TEAM_SHARED = 1, TEAM_NODE = 2, TEAM_SAME_MYPE_NODE = 3, TEAM_SAME_GPU = 4, TEAM_GPU_LEADERS = 5, TEAM_FIRST_USER = 6 };

// ---- small helpers that work for both heap back ends
static int local_write(void* dst, const void* src, size_t n) {
  Runtime& r = rt();
  if (!r.have_gpu) { memcpy(dst, src, n); return 0; }
  return cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : 1;
}
static int local_read(void* dst, const void* src, size_t n) {
  Runtime& r = rt();
  if (!r.have_gpu) { memcpy(dst, src, n); return 0; }
  return cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
static int local_zero(void* dst, size_t n) {
  Runtime& r = rt();
  if (!r.have_gpu) { memset(dst, 0, n); return 0; }
  return cudaMemset(dst, 0, n) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess ? 0 : 1;
}

Team* team_get(int handle) {
  Runtime& r = rt();
  if (handle < 0 || handle >= (int)r.teams.size()) return nullptr;
  return r.teams[handle].get();
}

void team_sync_ptrs(const Runtime& r, int idx, uint64_t* sync, uint64_t* ll, uint64_t* scratch, uint64_t* ll128) {
  size_t per = r.sync_bytes + r.ll_bytes + 2 * r.scratch_bytes + r.ll128_bytes;
  char* base = r.team_area + (size_t)idx * per;
  *sync = (uint64_t)base;
  *ll = (uint64_t)(base + r.sync_bytes);
  *scratch = (uint64_t)(base + r.sync_bytes + r.ll_bytes);
  if (ll128) *ll128 = (uint64_t)(base + r.sync_bytes + r.ll_bytes + 2 * r.scratch_bytes);
}

static bool bitmap_test(const std::vector<uint64_t>& b, int i) { return (b[i / 64] >> (i % 64)) & 1; }
static void bitmap_set(std::vector<uint64_t>& b, int i, bool free_) {
  if (free_) b[i / 64] |= 1ull << (i % 64);
  else b[i / 64] &= ~(1ull << (i % 64));
}

// Writes team `t` into slot t->idx of the device-visible pool.
static int publish_team(Runtime& r, Team* t) {
  bshmemi_team_t d{};
  d.my_pe = t->my_pe;
  d.start = t->start;
  d.stride = t->stride;
  d.size = t->size;
  d.team_idx = t->idx;
  d.has_nvls = t->nvls;
  d.mc_base = t->nvls ? (uint64_t)t->mc_base : 0;
  team_sync_ptrs(r, t->idx, &d.sync_base, &d.ll_base, &d.scratch_base, &d.ll128_base);
  d.scratch_bytes = r.scratch_bytes;
  d.ll_bytes = r.ll_bytes;
  d.ll128_bytes = r.ll128_bytes;
  d.epochs = (uint64_t)(r.epochs_dev + (size_t)t->idx * 2 * BSHMEM_SYNC_SLOTS);
  d.pe_of = 0;
  if (!t->strided) {
    if (r.have_gpu) {
      if (cudaMalloc((void**)&t->pe_of_dev, sizeof(int32_t) * t->size) != cudaSuccess) return ST_OUT_OF_MEMORY;
      cudaMemcpy(t->pe_of_dev, t->members.data(), sizeof(int32_t) * t->size, cudaMemcpyHostToDevice);
    } else {
      t->pe_of_dev = new int32_t[t->size];
      memcpy(t->pe_of_dev, t->members.data(), sizeof(int32_t) * t->size);
    }
    d.pe_of = (uint64_t)t->pe_of_dev;
  }
  r.team_pool_host[t->idx] = d;
  return local_write(r.team_pool_dev + t->idx, &d, sizeof(d)) ? ST_INTERNAL : ST_SUCCESS;
}

// After the heap's multicast window changed (it went away, or moved): rewrites the NVLS fields of every team.
void teams_refresh_nvls(Runtime& r) {
  char* world_mc = r.heap->mc_base();
  for (auto& up : r.teams) {
    Team* t = up.get();
    if (!t || t->idx < 0) continue;
    if (!world_mc) {  // the heap dropped every multicast object, the teams' own windows included
      t->nvls = false;
      t->mc_id = -1;
      t->mc_base = nullptr;
      t->mc_bytes = 0;
    } else if (t->nvls && t->mc_id < 0) {
      t->mc_base = world_mc;
      t->mc_bytes = r.heap->backed();
    }
    bshmemi_team_t& d = r.team_pool_host[t->idx];
    const uint64_t mc = t->nvls ? (uint64_t)t->mc_base : 0;
    if (d.has_nvls == (t->nvls ? 1 : 0) && d.mc_base == mc) continue;
    d.has_nvls = t->nvls;
    d.mc_base = mc;
    local_write(r.team_pool_dev + t->idx, &d, sizeof(d));
  }
}

// A team's own window was made for the heap as it was backed then.  Growth is a step of all PEs, so every
// member gives its window up here, at the same point of the program; the team goes on with the
// peer-to-peer algorithms.  Teams that use the world's window follow the heap and are not touched.
void teams_drop_windows(Runtime& r) {
  int dropped = 0;
  for (auto& up : r.teams) {
    Team* t = up.get();
    if (!t || t->mc_id < 0) continue;
    r.heap->team_mc_drop(t->mc_id);
    t->mc_id = -1;
    t->nvls = false;
    t->mc_base = nullptr;
    t->mc_bytes = 0;
    ++dropped;
  }
  if (dropped) WARN("the symmetric heap grew: %d team multicast window(s) were given up (size the heap with NVSHMEM_SYMMETRIC_SIZE before making teams to keep them)", dropped);
  teams_refresh_nvls(r);
}

static Team* install_team(Runtime& r, int idx, int start, int stride, int size, const std::vector<int>* members, int parent) {
  auto t = std::make_unique<Team>();
  t->idx = idx;
  t->start = start;
  t->stride = stride;
  t->size = size;
  t->parent = parent;
  if (members) {
    t->members = *members;
    t->strided = false;
    // An arithmetic progression is stored as a strided team all the same.
    bool ap = true;
    int st = size > 1 ? (*members)[1] - (*members)[0] : 1;
    for (int i = 1; i < size && ap; ++i) ap = (*members)[i] - (*members)[i - 1] == st;
    if (ap && st > 0) { t->strided = true; t->start = (*members)[0]; t->stride = st; }
  } else {
    for (int i = 0; i < size; ++i) t->members.push_back(start + i * stride);
  }
  auto it = std::find(t->members.begin(), t->members.end(), r.mype);
  t->my_pe = it == t->members.end() ? -1 : (int)(it - t->members.begin());
  // The world multicast window sums over every PE, so only teams that span the
  // world in world order may use it.
  t->nvls = r.heap->mc_base() != nullptr && size == r.npes && t->strided && t->start == 0 && t->stride == 1;
  if (t->nvls) {
    t->mc_base = r.heap->mc_base();
    t->mc_bytes = r.heap->backed();
  }
  if ((int)r.teams.size() <= idx) r.teams.resize(idx + 1);
  r.teams[idx] = std::move(t);
  bitmap_set(r.team_bitmap, idx, false);
  return r.teams[idx].get();
}

int teams_init(Runtime& r) {
  const Options& o = options();
  r.sync_bytes = round_up((size_t)BSHMEM_SYNC_SLOTS * r.npes * sizeof(uint64_t), 512);
  // Flag-in-data packets double the payload; two generations avoid a reset barrier.
  r.ll_bytes = round_up(2 * 2 * std::max<size_t>(o.FCOLLECT_LL_THRESHOLD, 2048) * r.npes, 512);
  r.scratch_bytes = round_up(std::max<size_t>(o.REDUCE_SCRATCH_SIZE, 4096), 512);
  // 128-byte packets: two generations of [npes][P] lines for fcollect / allreduce, two of [P] lines for broadcast and
  // npes acknowledgement words, P = packets of the largest message (120 payload bytes per line).
  const size_t p128 = (o.LL128_THRESHOLD + 119) / 120;
  r.ll128_bytes = p128 ? round_up(2 * 128 * p128 * ((size_t)r.npes + 1) + 8 * (size_t)r.npes, 512) : 0;
  size_t per = r.sync_bytes + r.ll_bytes + 2 * r.scratch_bytes + r.ll128_bytes;
  const int words = (r.max_teams + 63) / 64;
  r.team_area_bytes = per * r.max_teams;
  int hst = 0;
  r.team_area = (char*)r.heap->allocate(r.team_area_bytes, 4096, &hst);
  // Mail slots for internal agreement: [npes][8] uint64 written by peers, plus reduction buffers.
  r.host_scratch64 = (uint64_t*)r.heap->allocate(sizeof(uint64_t) * ((size_t)r.npes * 8 + 4 * words + 8), 512, &hst);
  if (!r.team_area || !r.host_scratch64) {
    ERROR_PRINT("cannot allocate the team area (%zu bytes)", r.team_area_bytes);
    return ST_OUT_OF_MEMORY;
  }
  if (local_zero(r.team_area, r.team_area_bytes) || local_zero(r.host_scratch64, sizeof(uint64_t) * ((size_t)r.npes * 8 + 4 * words + 8))) return ST_INTERNAL;

  r.team_pool_host.assign(r.max_teams, bshmemi_team_t{});
  for (auto& t : r.team_pool_host) { t.my_pe = -1; t.team_idx = -1; }
  size_t epoch_words = (size_t)r.max_teams * 2 * BSHMEM_SYNC_SLOTS;
  if (r.have_gpu) {
    if (cudaMalloc((void**)&r.team_pool_dev, sizeof(bshmemi_team_t) * r.max_teams) != cudaSuccess) return ST_OUT_OF_MEMORY;
    if (cudaMalloc((void**)&r.epochs_dev, sizeof(uint64_t) * epoch_words) != cudaSuccess) return ST_OUT_OF_MEMORY;
    cudaMemset(r.epochs_dev, 0, sizeof(uint64_t) * epoch_words);
    cudaMemcpy(r.team_pool_dev, r.team_pool_host.data(), sizeof(bshmemi_team_t) * r.max_teams, cudaMemcpyHostToDevice);
  } else {
    r.team_pool_dev = new bshmemi_team_t[r.max_teams];
    memcpy(r.team_pool_dev, r.team_pool_host.data(), sizeof(bshmemi_team_t) * r.max_teams);
    r.epochs_dev = new uint64_t[epoch_words]();
  }
  r.dstate.team_pool = (uint64_t)r.team_pool_dev;
  r.team_bitmap.assign(words, ~0ull);
  for (int i = r.max_teams; i < words * 64; ++i) bitmap_set(r.team_bitmap, i, false);

  // ---- predefined teams
  std::vector<int> node, same_mype, same_gpu, leaders;
  const PeInfo& me = r.pe_info[r.mype];
  std::vector<int> node_rank(r.npes, 0);
  for (int pe = 0; pe < r.npes; ++pe) {
    int k = 0;
    for (int q = 0; q < pe; ++q) k += r.pe_info[q].host_hash == r.pe_info[pe].host_hash;
    node_rank[pe] = k;
  }
  for (int pe = 0; pe < r.npes; ++pe) {
    const PeInfo& p = r.pe_info[pe];
    if (p.host_hash == me.host_hash) node.push_back(pe);
    if (node_rank[pe] == node_rank[r.mype]) same_mype.push_back(pe);
    if (p.host_hash == me.host_hash && memcmp(p.uuid, me.uuid, 16) == 0) same_gpu.push_back(pe);
    bool leader = true;
    for (int q = 0; q < pe; ++q)
      if (r.pe_info[q].host_hash == p.host_hash && memcmp(r.pe_info[q].uuid, p.uuid, 16) == 0) leader = false;
    if (leader) leaders.push_back(pe);
  }
  Team* t = install_team(r, TEAM_WORLD, 0, 1, r.npes, nullptr, -1);
  if (publish_team(r, t)) return ST_INTERNAL;
  const std::vector<int>* sets[] = {&node, &node, &same_mype, &same_gpu, &leaders};
  for (int i = 0; i < 5; ++i) {
    t = install_team(r, TEAM_SHARED + i, (*sets[i])[0], 1, (int)sets[i]->size(), sets[i], TEAM_WORLD);
    if (publish_team(r, t)) return ST_INTERNAL;
  }
  INFO(SUB_TEAM, "team area: %d slots x %zu bytes (sync %zu, LL %zu, scratch 2x%zu, LL128 %zu)", r.max_teams, per, r.sync_bytes, r.ll_bytes, r.scratch_bytes, r.ll128_bytes);
  return ST_SUCCESS;
}

void teams_finalize(Runtime& r) {
  for (auto& t : r.teams) {
    if (!t || !t->pe_of_dev) continue;
    if (r.have_gpu) cudaFree(t->pe_of_dev);
    else delete[] t->pe_of_dev;
  }
  r.teams.clear();
  if (r.have_gpu) {
    if (r.team_pool_dev) cudaFree(r.team_pool_dev);
    if (r.epochs_dev) cudaFree(r.epochs_dev);
  } else {
    delete[] r.team_pool_dev;
    delete[] r.epochs_dev;
  }
  r.team_pool_dev = nullptr;
  r.epochs_dev = nullptr;
  r.team_area = nullptr;
  r.host_scratch64 = nullptr;
}

int team_translate_pe(int src_team, int src_pe, int dst_team) {
  Team* s = team_get(src_team);
  Team* d = team_get(dst_team);
  if (!s || !d || src_pe < 0 || src_pe >= s->size) return -1;
  int world = s->members[src_pe];
  auto it = std::find(d->members.begin(), d->members.end(), world);
  return it == d->members.end() ? -1 : (int)(it - d->members.begin());
}

// AND-reduces `words` uint64 over the members of `team`; every member gets the result.
static int team_and_reduce(int team, uint64_t* data, int words);

// Picks the lowest team index that is free on every member of `parent`.
static int agree_on_index(int parent, int* idx_out) {
  Runtime& r = rt();
  std::vector<uint64_t> bits = r.team_bitmap;
  int st = team_and_reduce(parent, bits.data(), (int)bits.size());
  if (st != ST_SUCCESS) return st;
  for (int i = TEAM_FIRST_USER; i < r.max_teams; ++i)
    if (bitmap_test(bits, i)) {
      *idx_out = i;
      return ST_SUCCESS;
    }
  ERROR_PRINT("no free team slot (NVSHMEM_MAX_TEAMS=%d)", r.max_teams);
  return ST_OUT_OF_MEMORY;
}

// Gives team `t` (just installed, not yet published) an NVLink multicast window of its own: an object that the
// team's first member creates, that every member joins with its device and binds its part of the heap to.
// Every member of `parent` calls this, members of the new team or not, because the three agreements
// (created / all joined / all bound) run over the parent: after a failure anywhere nobody waits for anybody,
// everyone undoes its part and the team uses the peer-to-peer algorithms
// (reference: src/host/team/team_internal.cpp:749-851).
static int team_window_setup(Runtime& r, int parent, Team* t, int idx, const std::vector<int>& members) {
  const bool member = t != nullptr;
  int id = -1;
  uint64_t ok = ~0ull;
  if (member) {
    int live = 0;
    for (auto& up : r.teams) live += up && up->mc_id >= 0;
    if (live >= (int)options().NVLS_TEAM_WINDOWS || r.heap->team_mc_create(members, (uint32_t)idx, &id) != HEAP_OK) ok = 0;
  }
  int st = team_and_reduce(parent, &ok, 1);
  if (st != ST_SUCCESS) return st;
  if (ok && member && r.heap->team_mc_join(id, (int)options().BOOTSTRAP_TIMEOUT_MS) != HEAP_OK) ok = 0;
  if (ok) {
    st = team_and_reduce(parent, &ok, 1);
    if (st != ST_SUCCESS) return st;
  }
  char* base = nullptr;
  size_t bytes = 0;
  if (ok && member && r.heap->team_mc_bind(id, &base, &bytes) != HEAP_OK) ok = 0;
  if (ok) {
    st = team_and_reduce(parent, &ok, 1);
    if (st != ST_SUCCESS) return st;
  }
  if (!member) return ST_SUCCESS;
  if (!ok) {
    r.heap->team_mc_drop(id);
    return ST_SUCCESS;
  }
  t->nvls = true;
  t->mc_id = id;
  t->mc_base = base;
  t->mc_bytes = bytes;
  return ST_SUCCESS;
}

int team_create_from_members(int parent, const std::vector<int>& world_members, uint64_t uniqueid, int* new_team) {
  Runtime& r = rt();
  *new_team = BSHMEM_TEAM_INVALID;
  int idx = -1;
  int st = agree_on_index(parent, &idx);
  if (st != ST_SUCCESS) return st;
  bool member = std::find(world_members.begin(), world_members.end(), r.mype) != world_members.end();
  Team* t = nullptr;
  if (member) {
    t = install_team(r, idx, world_members[0], 1, (int)world_members.size(), &world_members, parent);
    t->uniqueid = uniqueid;
  }
  // A team that spans the world in world order shares the world's window (install_team); any other team of
  // two or more PEs gets a window of its own where the heap has NVLS.  All inputs of this decision are the
  // same on every member of the parent.
  bool spans_world = (int)world_members.size() == r.npes;
  for (int i = 0; i < (int)world_members.size() && spans_world; ++i) spans_world = world_members[i] == i;
  if (r.have_gpu && r.heap->mc_base() && world_members.size() >= 2 && !spans_world && options().NVLS_TEAM_WINDOWS > 0) {
    st = team_window_setup(r, parent, t, idx, world_members);
    if (st != ST_SUCCESS) return st;
  }
  if (member) {
    st = publish_team(r, t);
    if (st != ST_SUCCESS) return st;
    *new_team = idx;
  }
  // Nobody uses the new team before every member has published it.
  return host_sync_team(parent, r.stream, true);
}

int team_split_strided(int parent, int start, int stride, int size, uint64_t uniqueid, int num_contexts, int* new_team) {
  Team* p = team_get(parent);
  *new_team = BSHMEM_TEAM_INVALID;
  if (!p || p->my_pe < 0) return ST_INVALID_VALUE;
  if (size <= 0 || start < 0 || start >= p->size || (size > 1 && stride == 0)) return ST_INVALID_VALUE;
  long last = (long)start + (long)(size - 1) * stride;
  if (last < 0 || last >= p->size) return ST_INVALID_VALUE;
  std::vector<int> members;
  for (int i = 0; i < size; ++i) members.push_back(p->members[start + i * stride]);
  (void)num_contexts;
  return team_create_from_members(parent, members, uniqueid, new_team);
}

int team_split_2d(int parent, int xrange, int* xteam, int* yteam) {
  Team* p = team_get(parent);
  *xteam = *yteam = BSHMEM_TEAM_INVALID;
  if (!p || p->my_pe < 0 || xrange <= 0) return ST_INVALID_VALUE;
  if (xrange > p->size) xrange = p->size;
  const int n = p->size, me = p->my_pe;
  const int rows = (n + xrange - 1) / xrange;
  // x teams: consecutive runs of `xrange` parent PEs; one collective step per row
  // so that every parent member takes part in every agreement.
  for (int row = 0; row < rows; ++row) {
    int s = row * xrange, sz = std::min(xrange, n - s), nt;
    int st = team_split_strided(parent, s, 1, sz, 0, 0, &nt);
    if (st != ST_SUCCESS) return st;
    if (me / xrange == row) *xteam = nt;
  }
  // y teams: same column of every row.
  for (int col = 0; col < xrange; ++col) {
    int sz = (n - col + xrange - 1) / xrange, nt;
    if (sz <= 0) continue;
    int st = team_split_strided(parent, col, xrange, sz, 0, 0, &nt);
    if (st != ST_SUCCESS) return st;
    if (me % xrange == col) *yteam = nt;
  }
  return ST_SUCCESS;
}

int team_destroy(int handle) {
  Runtime& r = rt();
  Team* t = team_get(handle);
  if (!t || handle < TEAM_FIRST_USER) return ST_INVALID_VALUE;
  // Every member has left its last collective on this team once the barrier
  // completes; after that the slot's flags and epochs can be cleared.
  int st = host_barrier_team(handle, r.stream, true);
  if (st != ST_SUCCESS) return st;
  for (int c : t->children) team_destroy(c);
  uint64_t sync, ll, scratch, ll128;
  team_sync_ptrs(r, handle, &sync, &ll, &scratch, &ll128);
  // The whole slot: sync flags, flag-in-data packets, both scratch halves (the recursive exchange keeps round flags
  // there, compared against the team's generation, which restarts at zero for the slot's next team), LL128 lines.
  local_zero((void*)sync, r.sync_bytes + r.ll_bytes + 2 * r.scratch_bytes + r.ll128_bytes);
  (void)ll;
  (void)scratch;
  (void)ll128;
  local_zero(r.epochs_dev + (size_t)handle * 2 * BSHMEM_SYNC_SLOTS, sizeof(uint64_t) * 2 * BSHMEM_SYNC_SLOTS);
  bshmemi_team_t blank{};
  blank.my_pe = -1;
  blank.team_idx = -1;
  r.team_pool_host[handle] = blank;
  local_write(r.team_pool_dev + handle, &blank, sizeof(blank));
  if (t->pe_of_dev) {
    if (r.have_gpu) cudaFree(t->pe_of_dev);
    else delete[] t->pe_of_dev;
  }
  if (t->mc_id >= 0) r.heap->team_mc_drop(t->mc_id);
  r.teams[handle].reset();
  bitmap_set(r.team_bitmap, handle, true);
  return ST_SUCCESS;
}

// ------------------------------------------------------------------ AND reduction
// Used only on the control path (team creation).  GPU heap: each member writes
// its words into every member's mail slot with peer copies, a team sync orders
// them, then each member combines its own slots locally.  Host heap: the same
// through plain memory.
static int team_and_reduce(int team, uint64_t* data, int words) {
  Runtime& r = rt();
  Team* t = team_get(team);
  if (!t || t->my_pe < 0) return ST_INVALID_VALUE;
  if (t->size == 1) return ST_SUCCESS;
  if (words > 6) return ST_INVALID_VALUE;  // mail slot: 8 words, two are header
  if (!r.have_gpu) return emul_allreduce_and_u64(team, data, words);
  uint64_t msg[8] = {0};
  memcpy(msg, data, sizeof(uint64_t) * words);
  for (int i = 0; i < t->size; ++i) {
    uint64_t* remote = (uint64_t*)r.heap->translate(r.host_scratch64 + (size_t)r.mype * 8, t->members[i]);
    if (cudaMemcpyAsync(remote, msg, sizeof(msg), cudaMemcpyHostToDevice, r.stream) != cudaSuccess) return ST_INTERNAL;
  }
  // Barrier (not just sync): the copies above must have landed everywhere.
  int st = host_barrier_team(team, r.stream, true);
  if (st != ST_SUCCESS) return st;
  for (int i = 0; i < t->size; ++i) {
    uint64_t got[8];
    if (local_read(got, r.host_scratch64 + (size_t)t->members[i] * 8, sizeof(got))) return ST_INTERNAL;
    for (int w = 0; w < words; ++w) data[w] &= got[w];
  }
  // Slots may be rewritten by the next agreement only after everyone has read them.
  return host_sync_team(team, r.stream, true);
}

}  // namespace bshmem
