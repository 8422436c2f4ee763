// UID bootstrap: a TCP rendezvous that needs no launcher support.
//
// One process asks for a unique id.  That call picks a listen address, draws a
// 64-bit magic from /dev/urandom and starts a detached *root thread*.  The id
// (version, magic, root address) reaches the other processes out of band
// (torch.distributed broadcast, a file, MPI ...).  Every rank then opens its own
// listen socket, registers {rank, nranks, listen address} with the root and
// gets the complete address table back.  Peer connections are made lazily, one
// persistent socket per pair (the lower rank connects, the higher accepts), and
// carry three collectives: ring allgather, pairwise alltoall and a
// dissemination barrier.  Every blocking step has a deadline
// (NVSHMEM_BOOTSTRAP_TIMEOUT_MS) and reports a status; nothing calls exit()
// (reference behaviour: src/modules/bootstrap/uid/bootstrap_uid.cpp).
#include <fcntl.h>
#include <pthread.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "../util/env.h"
#include "../util/log.h"
#include "bootstrap.h"
#include "socket.h"

namespace bshmem {

namespace {

constexpr uint32_t kWireVersion = 0xB2000001u;

struct IdPayload {  // lives in bshmem_uniqueid_t::internal
  uint64_t magic;
  SockAddr root;
};
static_assert(sizeof(IdPayload) <= sizeof(((bshmem_uniqueid_t*)0)->internal), "unique id too small");

struct Registration {
  uint32_t wire_version;
  uint32_t rank;
  uint32_t nranks;
  uint32_t pad;
  SockAddr listen;
};

struct RootReply {
  uint32_t status;  // BootstrapStatus
  uint32_t nranks;
};

std::atomic<int> g_test_drop_rank{-1};

uint64_t random_u64() {
  uint64_t v = 0;
  int fd = open("/dev/urandom", O_RDONLY | O_CLOEXEC);
  if (fd >= 0) {
    ssize_t r = read(fd, &v, sizeof(v));
    (void)r;
    close(fd);
  }
  if (v == 0) v = ((uint64_t)getpid() << 32) ^ (uint64_t)time(nullptr) ^ 0x9e3779b97f4a7c15ull;
  return v;
}

int timeout_ms() { return (int)options().BOOTSTRAP_TIMEOUT_MS; }

// ---------------------------------------------------------------- root thread
struct RootArgs {
  int listen_fd;
  uint64_t magic;
  int timeout_ms;  // read by the creating thread: the root thread never touches the option table (it may be reloaded meanwhile)
};

void root_main(RootArgs args) {
  pthread_setname_np(pthread_self(), "bshmem-uidroot");
  const int tmo = args.timeout_ms;
  std::vector<int> fds;
  std::vector<SockAddr> table;
  std::vector<bool> seen;
  uint32_t nranks = 0, arrived = 0;
  uint32_t status = BOOT_OK;
  while (nranks == 0 || arrived < nranks) {
    int fd = -1;
    int st = sock_accept(args.listen_fd, args.magic, tmo, &fd);
    if (st == SOCK_BAD_MAGIC) continue;  // a stray connection; keep waiting
    if (st != SOCK_OK) {
      WARN("UID root: gave up waiting for ranks (%u of %u registered): %s", arrived, nranks, sock_strerror(st));
      status = BOOT_ERR_TIMEOUT;
      break;
    }
    Registration reg;
    if (sock_recv(fd, &reg, sizeof(reg), tmo) != SOCK_OK) { sock_close(fd); continue; }
    if (reg.wire_version != kWireVersion) {
      RootReply rep{BOOT_ERR_VERSION, 0};
      sock_send(fd, &rep, sizeof(rep), tmo);
      sock_close(fd);
      status = BOOT_ERR_VERSION;
      break;
    }
    if (nranks == 0) {
      nranks = reg.nranks;
      fds.assign(nranks, -1);
      table.resize(nranks);
      seen.assign(nranks, false);
    }
    if (reg.nranks != nranks || reg.rank >= nranks || seen[reg.rank]) {
      RootReply rep{BOOT_ERR_ARGS, 0};
      sock_send(fd, &rep, sizeof(rep), tmo);
      sock_close(fd);
      status = BOOT_ERR_ARGS;
      break;
    }
    if ((int)reg.rank == g_test_drop_rank.load()) {  // host-side fault injection
      sock_close(fd);
      continue;
    }
    seen[reg.rank] = true;
    fds[reg.rank] = fd;
    table[reg.rank] = reg.listen;
    ++arrived;
  }
  for (uint32_t r = 0; r < fds.size(); ++r) {
    if (fds[r] < 0) continue;
    RootReply rep{status, nranks};
    if (sock_send(fds[r], &rep, sizeof(rep), tmo) == SOCK_OK && status == BOOT_OK)
      sock_send(fds[r], table.data(), table.size() * sizeof(SockAddr), tmo);
    sock_close(fds[r]);
  }
  sock_close(args.listen_fd);
}

int start_root(SockAddr* addr, uint64_t magic) {
  int fd = -1;
  if (sock_listen(addr, &fd) != SOCK_OK) return BOOT_ERR_SOCKET;
  std::thread(root_main, RootArgs{fd, magic, timeout_ms()}).detach();
  return BOOT_OK;
}

// ---------------------------------------------------------------- per-rank state
struct UidState {
  int rank = 0, nranks = 0;
  uint64_t magic = 0;
  int listen_fd = -1;
  std::vector<SockAddr> table;
  std::map<int, int> conn;     // peer rank -> fd
  std::mutex mu;
  volatile int abort_flag = 0;
};

int peer_fd(UidState* s, int peer, int* fd_out) {
  auto it = s->conn.find(peer);
  if (it != s->conn.end()) { *fd_out = it->second; return BOOT_OK; }
  const int tmo = timeout_ms();
  if (s->rank < peer) {
    int fd = -1;
    int st = sock_connect(s->table[peer], s->magic, tmo, &fd, &s->abort_flag);
    if (st != SOCK_OK) return st == SOCK_TIMEOUT ? BOOT_ERR_TIMEOUT : BOOT_ERR_SOCKET;
    uint32_t me = (uint32_t)s->rank;
    if (sock_send(fd, &me, sizeof(me), tmo) != SOCK_OK) { sock_close(fd); return BOOT_ERR_SOCKET; }
    s->conn[peer] = fd;
    *fd_out = fd;
    return BOOT_OK;
  }
  // Higher rank: accept until the wanted peer shows up; park the others.
  for (;;) {
    int fd = -1;
    int st = sock_accept(s->listen_fd, s->magic, tmo, &fd, &s->abort_flag);
    if (st == SOCK_BAD_MAGIC) continue;
    if (st != SOCK_OK) return st == SOCK_TIMEOUT ? BOOT_ERR_TIMEOUT : BOOT_ERR_SOCKET;
    uint32_t who = 0;
    if (sock_recv(fd, &who, sizeof(who), tmo) != SOCK_OK || who >= (uint32_t)s->nranks) { sock_close(fd); continue; }
    s->conn[(int)who] = fd;
    if ((int)who == peer) { *fd_out = fd; return BOOT_OK; }
  }
}

int map_sock(int st) {
  if (st == SOCK_OK) return BOOT_OK;
  if (st == SOCK_TIMEOUT) return BOOT_ERR_TIMEOUT;
  if (st == SOCK_CLOSED) return BOOT_ERR_PEER;
  return BOOT_ERR_SOCKET;
}

int uid_exchange(UidState* s, int to, const void* sbuf, size_t slen, int from, void* rbuf, size_t rlen) {
  int sfd = -1, rfd = -1;
  // Open the two connections in a fixed (rank) order so that a connect is never
  // stuck behind an accept on both ends of a pair.
  int first = std::min(to, from), second = std::max(to, from);
  int tmp;
  int st = peer_fd(s, first, &tmp);
  if (st != BOOT_OK) return st;
  st = peer_fd(s, second, &tmp);
  if (st != BOOT_OK) return st;
  peer_fd(s, to, &sfd);
  peer_fd(s, from, &rfd);
  return map_sock(sock_exchange(sfd, sbuf, slen, rfd, rbuf, rlen, timeout_ms()));
}

int uid_allgather(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  auto* s = (UidState*)h->comm_state;
  std::lock_guard<std::mutex> lk(s->mu);
  char* out = (char*)recvbuf;
  const int n = s->nranks, me = s->rank;
  if (sendbuf != out + (size_t)me * bytes) memcpy(out + (size_t)me * bytes, sendbuf, bytes);
  if (n == 1 || bytes == 0) return BOOT_OK;
  const int next = (me + 1) % n, prev = (me - 1 + n) % n;
  for (int step = 0; step < n - 1; ++step) {  // ring: forward the block received last
    int sblk = (me - step + n) % n, rblk = (me - step - 1 + n) % n;
    int st = uid_exchange(s, next, out + (size_t)sblk * bytes, bytes, prev, out + (size_t)rblk * bytes, bytes);
    if (st != BOOT_OK) return st;
  }
  return BOOT_OK;
}

int uid_alltoall(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  auto* s = (UidState*)h->comm_state;
  std::lock_guard<std::mutex> lk(s->mu);
  const char* in = (const char*)sendbuf;
  char* out = (char*)recvbuf;
  const int n = s->nranks, me = s->rank;
  memcpy(out + (size_t)me * bytes, in + (size_t)me * bytes, bytes);
  for (int d = 1; d < n; ++d) {  // pairwise: talk to rank+d while hearing from rank-d
    int to = (me + d) % n, from = (me - d + n) % n;
    int st = uid_exchange(s, to, in + (size_t)to * bytes, bytes, from, out + (size_t)from * bytes, bytes);
    if (st != BOOT_OK) return st;
  }
  return BOOT_OK;
}

int uid_barrier(bshmem_bootstrap_handle_t* h) {
  auto* s = (UidState*)h->comm_state;
  std::lock_guard<std::mutex> lk(s->mu);
  const int n = s->nranks, me = s->rank;
  for (int d = 1; d < n; d <<= 1) {  // dissemination: ceil(log2 n) rounds
    char tok = 1, got = 0;
    int st = uid_exchange(s, (me + d) % n, &tok, 1, (me - d % n + n) % n, &got, 1);
    if (st != BOOT_OK) return st;
  }
  return BOOT_OK;
}

void uid_global_exit(int status, bshmem_bootstrap_handle_t* h) {
  // Peers blocked in a bootstrap collective see their socket close and return
  // BOOT_ERR_PEER; this process leaves at once.
  auto* s = (UidState*)h->comm_state;
  if (s) {
    s->abort_flag = 1;
    for (auto& kv : s->conn) sock_close(kv.second);
    sock_close(s->listen_fd);
  }
  _exit(status);
}

int uid_finalize(bshmem_bootstrap_handle_t* h) {
  auto* s = (UidState*)h->comm_state;
  if (!s) return BOOT_OK;
  for (auto& kv : s->conn) sock_close(kv.second);
  sock_close(s->listen_fd);
  delete s;
  h->comm_state = nullptr;
  return BOOT_OK;
}

int uid_show_info(bshmem_bootstrap_handle_t* h) {
  auto* s = (UidState*)h->comm_state;
  INFO(SUB_BOOTSTRAP, "UID bootstrap: rank %d of %d, listening on %s, %zu peer connections", s->rank, s->nranks,
       s->table[s->rank].str().c_str(), s->conn.size());
  return BOOT_OK;
}

}  // namespace

void bootstrap_uid_test_drop_rank(int r) { g_test_drop_rank.store(r); }

const char* bootstrap_strerror(int st) {
  switch (st) {
    case BOOT_OK: return "ok";
    case BOOT_ERR_SOCKET: return "socket failure";
    case BOOT_ERR_TIMEOUT: return "timed out waiting for a peer";
    case BOOT_ERR_VERSION: return "bootstrap wire version mismatch";
    case BOOT_ERR_ARGS: return "inconsistent rank/nranks arguments";
    case BOOT_ERR_PEER: return "a peer closed its connection";
    case BOOT_ERR_PLUGIN: return "bootstrap plugin could not be loaded";
    default: return "unknown bootstrap error";
  }
}

int bootstrap_uid_get_unique_id(bshmem_uniqueid_t* id) {
  if (!id) return BOOT_ERR_ARGS;
  const Options& o = options();
  memset(id, 0, sizeof(*id));
  IdPayload p{};
  p.magic = random_u64();
  std::string ifname;
  if (!o.BOOTSTRAP_UID_SESSION_ID.empty()) {
    if (!sock_parse_hostport(o.BOOTSTRAP_UID_SESSION_ID, &p.root)) return BOOT_ERR_ARGS;
    p.magic = 0x5e5510ull;  // every rank derives the same magic from the session id
    for (char c : o.BOOTSTRAP_UID_SESSION_ID) p.magic = p.magic * 1099511628211ull ^ (uint8_t)c;
  } else {
    sock_pick_address(o.BOOTSTRAP_UID_SOCK_IFNAME, o.BOOTSTRAP_UID_SOCK_FAMILY, &p.root, &ifname);
  }
  int st = start_root(&p.root, p.magic);
  if (st != BOOT_OK) return st;
  INFO(SUB_BOOTSTRAP, "UID root listening on %s (%s)", p.root.str().c_str(), ifname.c_str());
  id->version = (int)((BSHMEM_BOOTSTRAP_ABI_VERSION << 16) + sizeof(bshmem_uniqueid_t));
  memcpy(id->internal, &p, sizeof(p));
  return BOOT_OK;
}

int bootstrap_uid_init(const bshmem_uniqueid_t* id, int rank, int nranks, bshmem_bootstrap_handle_t* h) {
  if (!h || nranks <= 0 || rank < 0 || rank >= nranks) return BOOT_ERR_ARGS;
  const Options& o = options();
  IdPayload p{};
  bshmem_uniqueid_t session_id;
  if (!id) {
    if (o.BOOTSTRAP_UID_SESSION_ID.empty()) return BOOT_ERR_ARGS;
    if (rank == 0) {
      int st = bootstrap_uid_get_unique_id(&session_id);
      if (st != BOOT_OK) return st;
      memcpy(&p, session_id.internal, sizeof(p));
    } else {
      if (!sock_parse_hostport(o.BOOTSTRAP_UID_SESSION_ID, &p.root)) return BOOT_ERR_ARGS;
      p.magic = 0x5e5510ull;
      for (char c : o.BOOTSTRAP_UID_SESSION_ID) p.magic = p.magic * 1099511628211ull ^ (uint8_t)c;
    }
  } else {
    if (id->version != (int)((BSHMEM_BOOTSTRAP_ABI_VERSION << 16) + sizeof(bshmem_uniqueid_t))) return BOOT_ERR_VERSION;
    memcpy(&p, id->internal, sizeof(p));
  }

  auto* s = new UidState();
  s->rank = rank;
  s->nranks = nranks;
  s->magic = p.magic;
  SockAddr mine;
  // Listen on the interface that can reach the root: same family, and the loopback
  // address when the root itself is on loopback.
  sock_pick_address(o.BOOTSTRAP_UID_SOCK_IFNAME, p.root.family == AF_INET6 ? "AF_INET6" : "AF_INET", &mine);
  bool root_is_loop = p.root.family == AF_INET ? p.root.addr[0] == 127 : (p.root.addr[15] == 1 && p.root.addr[0] == 0);
  if (root_is_loop) { memcpy(mine.addr, p.root.addr, 16); mine.scope_id = p.root.scope_id; }
  if (sock_listen(&mine, &s->listen_fd) != SOCK_OK) { delete s; return BOOT_ERR_SOCKET; }

  const int tmo = timeout_ms();
  // Spread the registrations of very large jobs so the root's backlog is not overrun.
  if (nranks > 128) usleep((rank % 128) * 1000);
  int rfd = -1;
  int st = sock_connect(p.root, p.magic, tmo, &rfd);
  if (st != SOCK_OK) { sock_close(s->listen_fd); delete s; return map_sock(st); }
  Registration reg{kWireVersion, (uint32_t)rank, (uint32_t)nranks, 0, mine};
  RootReply rep{};
  st = sock_send(rfd, &reg, sizeof(reg), tmo);
  if (st == SOCK_OK) st = sock_recv(rfd, &rep, sizeof(rep), tmo);
  int result = map_sock(st);
  if (result == BOOT_ERR_PEER) result = BOOT_ERR_TIMEOUT;  // the root gave up on the job
  if (result == BOOT_OK && rep.status != BOOT_OK) result = (int)rep.status;
  if (result == BOOT_OK && (int)rep.nranks != nranks) result = BOOT_ERR_ARGS;
  if (result == BOOT_OK) {
    s->table.resize(nranks);
    result = map_sock(sock_recv(rfd, s->table.data(), sizeof(SockAddr) * nranks, tmo));
  }
  sock_close(rfd);
  if (result != BOOT_OK) {
    sock_close(s->listen_fd);
    delete s;
    return result;
  }

  h->version = BSHMEM_BOOTSTRAP_ABI_VERSION;
  h->pg_rank = rank;
  h->pg_size = nranks;
  h->mype_node = rank;
  h->npes_node = nranks;
  h->allgather = uid_allgather;
  h->alltoall = uid_alltoall;
  h->barrier = uid_barrier;
  h->global_exit = uid_global_exit;
  h->finalize = uid_finalize;
  h->show_info = uid_show_info;
  h->comm_state = s;
  return BOOT_OK;
}

}  // namespace bshmem
