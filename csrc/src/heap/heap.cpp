#include "heap.h"

#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>

#include "../util/env.h"
#include "../util/log.h"

namespace bshmem {

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------ base class
void* SymmetricHeap::allocate(size_t size, size_t alignment, int* status) {
  if (status) *status = HEAP_OK;
  if (size == 0) return nullptr;
  // Nothing larger than the window can ever fit; refusing it here also keeps `size + alignment` below from wrapping.
  if (size > stride_ || alignment > stride_) {
    ERROR_PRINT("symmetric heap: request of %zu bytes (alignment %zu) exceeds the %zu-byte window (NVSHMEM_MAX_MEMORY_PER_GPU)", size, alignment, stride_);
    if (status) *status = HEAP_ERR_OOM;
    return nullptr;
  }
  size_t off = 0;
  if (!alloc_.allocate(size, alignment, &off)) {
    // Grow by the request plus its alignment slack, rounded to the growth granule.
    // Every PE takes this branch at the same call because the allocators are in
    // the same state, so `grow` can be collective.
    size_t need = round_up(size + (alignment > HeapAllocator::kMinAlign ? alignment : 0), granularity_);
    if (backed_ + need > stride_) {
      ERROR_PRINT("symmetric heap: request of %zu bytes exceeds the %zu-byte window (NVSHMEM_MAX_MEMORY_PER_GPU)", size, stride_);
      if (status) *status = HEAP_ERR_OOM;
      return nullptr;
    }
    int st = grow(need);
    if (st != HEAP_OK) {
      if (status) *status = st;
      return nullptr;
    }
    if (!alloc_.allocate(size, alignment, &off)) {
      if (status) *status = HEAP_ERR_OOM;
      return nullptr;
    }
  }
  return base() + off;
}

int SymmetricHeap::release(void* p) {
  if (!p) return HEAP_OK;
  if (!contains(p)) return HEAP_ERR_ARGS;
  return alloc_.release((size_t)((char*)p - base())) ? HEAP_OK : HEAP_ERR_ARGS;
}

size_t SymmetricHeap::allocation_size(const void* p) const {
  if (!contains(p)) return 0;
  return alloc_.size_of((size_t)((const char*)p - base()));
}

int SymmetricHeap::check_symmetry() {
  if (!boot_ || npes_ == 1) return HEAP_OK;
  std::vector<uint64_t> all(npes_);
  uint64_t mine = alloc_.history_digest();
  if (boot_->allgather(&mine, all.data(), sizeof(uint64_t), boot_) != 0) return HEAP_ERR_EXCHANGE;
  for (int pe = 0; pe < npes_; ++pe)
    if (all[pe] != mine) {
      ERROR_PRINT("symmetric heap: PE %d and PE %d made different allocation call sequences", mype_, pe);
      return HEAP_ERR_ASYMMETRIC;
    }
  return HEAP_OK;
}

// ------------------------------------------------------------------ FD exchange
static int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

static socklen_t make_name(sockaddr_un* sa, uint64_t key, int pe) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  // Abstract namespace (leading NUL): nothing is left behind in the file system.
  int n = snprintf(sa->sun_path + 1, sizeof(sa->sun_path) - 1, "bshmem-%016llx-%d", (unsigned long long)key, pe);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

FdExchange::~FdExchange() { close_all(); }

void FdExchange::close_all() {
  for (auto& p : pending_)
    if (p.fd >= 0) ::close(p.fd);
  pending_.clear();
  if (sock_ >= 0) ::close(sock_);
  sock_ = -1;
}

int FdExchange::open(uint64_t job_key, int mype, int npes) {
  key_ = job_key;
  mype_ = mype;
  npes_ = npes;
  sock_ = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock_ < 0) return HEAP_ERR_EXCHANGE;
  sockaddr_un sa;
  socklen_t len = make_name(&sa, key_, mype_);
  if (bind(sock_, (sockaddr*)&sa, len) != 0) {
    ERROR_PRINT("fd exchange: bind failed: %s", strerror(errno));
    ::close(sock_);
    sock_ = -1;
    return HEAP_ERR_EXCHANGE;
  }
  return HEAP_OK;
}

struct FdMsg {
  int32_t from;
  uint32_t seq;
};

int FdExchange::send_fd(int to_pe, int fd, uint32_t seq, int timeout_ms) {
  FdMsg body{mype_, seq};
  iovec iov{&body, sizeof(body)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  sockaddr_un sa;
  socklen_t len = make_name(&sa, key_, to_pe);
  msghdr msg{};
  msg.msg_name = &sa;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    ssize_t r = sendmsg(sock_, &msg, MSG_DONTWAIT | MSG_NOSIGNAL);
    if (r == (ssize_t)sizeof(body)) return HEAP_OK;
    // The peer's queue is full, or it has not bound its socket yet: retry until the deadline.
    if (errno != EAGAIN && errno != EWOULDBLOCK && errno != ECONNREFUSED && errno != ENOENT && errno != EINTR && errno != ENOBUFS) {
      ERROR_PRINT("fd exchange: sendmsg to PE %d failed: %s", to_pe, strerror(errno));
      return HEAP_ERR_EXCHANGE;
    }
    if (now_ms() > deadline) return HEAP_ERR_EXCHANGE;
    usleep(500);
  }
}

int FdExchange::recv_fd(int from_pe, uint32_t seq, int* fd_out, int timeout_ms) {
  int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    for (size_t i = 0; i < pending_.size(); ++i)
      if (pending_[i].from == from_pe && pending_[i].seq == seq) {
        *fd_out = pending_[i].fd;
        pending_.erase(pending_.begin() + i);
        return HEAP_OK;
      }
    int64_t left = deadline - now_ms();
    if (left <= 0) return HEAP_ERR_EXCHANGE;
    pollfd p{sock_, POLLIN, 0};
    int pr = poll(&p, 1, (int)std::min<int64_t>(left, 200));
    if (pr <= 0) continue;
    FdMsg body{};
    iovec iov{&body, sizeof(body)};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t r = recvmsg(sock_, &msg, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (r != (ssize_t)sizeof(body)) continue;
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) continue;
    int fd = -1;
    memcpy(&fd, CMSG_DATA(c), sizeof(int));
    pending_.push_back(Pending{body.from, body.seq, fd});
  }
}

int FdExchange::allgather_fd(int my_fd, uint32_t seq, std::vector<int>* out, int timeout_ms) {
  out->assign(npes_, -1);
  // One send and one receive per step keeps at most a couple of datagrams
  // queued per socket (the kernel's default queue is short).
  for (int d = 1; d < npes_; ++d) {
    int to = (mype_ + d) % npes_, from = (mype_ - d + npes_) % npes_;
    int st = send_fd(to, my_fd, seq, timeout_ms);
    if (st != HEAP_OK) return st;
    st = recv_fd(from, seq, &(*out)[from], timeout_ms);
    if (st != HEAP_OK) return st;
  }
  return HEAP_OK;
}

int FdExchange::bcast_fd(int root, int* fd_inout, uint32_t seq, int timeout_ms) {
  if (mype_ == root) {
    for (int pe = 0; pe < npes_; ++pe) {
      if (pe == root) continue;
      int st = send_fd(pe, *fd_inout, seq, timeout_ms);
      if (st != HEAP_OK) return st;
    }
    return HEAP_OK;
  }
  return recv_fd(root, seq, fd_inout, timeout_ms);
}

int FdExchange::bcast_fd_group(int root, const std::vector<int>& members, int* fd_inout, uint32_t seq, int timeout_ms) {
  if (mype_ == root) {
    for (int pe : members) {
      if (pe == root) continue;
      int st = send_fd(pe, *fd_inout, seq, timeout_ms);
      if (st != HEAP_OK) return st;
    }
    return HEAP_OK;
  }
  return recv_fd(root, seq, fd_inout, timeout_ms);
}

// ------------------------------------------------------------------ host-memory heap
namespace {

class HostHeap final : public SymmetricHeap {
 public:
  ~HostHeap() override { finalize(); }
  const char* kind() const override { return "HOST"; }
  bool device_memory() const override { return false; }

  int init(bshmem_bootstrap_handle_t* boot, int, size_t stride, size_t initial, size_t granularity) override {
    boot_ = boot;
    mype_ = boot->pg_rank;
    npes_ = boot->pg_size;
    long page = sysconf(_SC_PAGESIZE);
    granularity_ = round_up(std::max<size_t>(granularity, (size_t)page), (size_t)page);
    stride_ = round_up(stride, granularity_);
    // All PEs must agree on the shared-memory names: PE 0 draws a key.
    uint64_t key = 0;
    if (mype_ == 0) key = ((uint64_t)getpid() << 32) ^ (uint64_t)now_ms() ^ (uint64_t)(uintptr_t)this;
    std::vector<uint64_t> keys(npes_);
    if (boot->allgather(&key, keys.data(), sizeof(key), boot) != 0) return HEAP_ERR_EXCHANGE;
    key_ = keys[0];
    void* va = mmap(nullptr, stride_ * npes_, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (va == MAP_FAILED) {
      ERROR_PRINT("host heap: cannot reserve %zu bytes of address space: %s", stride_ * npes_, strerror(errno));
      return HEAP_ERR_OOM;
    }
    window_base_ = (char*)va;
    fds_.assign(npes_, -1);
    fd_ = shm_open(name(mype_).c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
    if (fd_ < 0) {
      ERROR_PRINT("host heap: shm_open(%s) failed: %s", name(mype_).c_str(), strerror(errno));
      return HEAP_ERR_DRIVER;
    }
    fds_[mype_] = fd_;
    if (boot->barrier(boot) != 0) return HEAP_ERR_EXCHANGE;  // every segment exists now
    for (int pe = 0; pe < npes_; ++pe) {
      if (pe == mype_) continue;
      fds_[pe] = shm_open(name(pe).c_str(), O_RDWR | O_CLOEXEC, 0600);
      if (fds_[pe] < 0) {
        ERROR_PRINT("host heap: cannot open the segment of PE %d: %s", pe, strerror(errno));
        return HEAP_ERR_EXCHANGE;
      }
    }
    if (boot->barrier(boot) != 0) return HEAP_ERR_EXCHANGE;
    shm_unlink(name(mype_).c_str());  // all peers hold descriptors; the name can go
    return grow(round_up(std::max<size_t>(initial, granularity_), granularity_));
  }

  int grow(size_t bytes) override {
    size_t new_size = backed_ + bytes;
    if (new_size > stride_) return HEAP_ERR_OOM;
    if (ftruncate(fd_, (off_t)new_size) != 0) {
      ERROR_PRINT("host heap: ftruncate to %zu failed: %s", new_size, strerror(errno));
      return HEAP_ERR_OOM;
    }
    if (boot_->barrier(boot_) != 0) return HEAP_ERR_EXCHANGE;  // every segment has its new length
    for (int pe = 0; pe < npes_; ++pe) {
      void* at = window_base_ + (size_t)pe * stride_ + backed_;
      void* r = mmap(at, bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fds_[pe], (off_t)backed_);
      if (r == MAP_FAILED) {
        ERROR_PRINT("host heap: mmap of PE %d's chunk failed: %s", pe, strerror(errno));
        return HEAP_ERR_DRIVER;
      }
    }
    alloc_.add_chunk(backed_, bytes);
    backed_ = new_size;
    ++nchunks_;
    INFO(SUB_MEM, "host heap grew to %zu bytes (%d chunks)", backed_, nchunks_);
    return boot_->barrier(boot_) == 0 ? HEAP_OK : HEAP_ERR_EXCHANGE;
  }

  int zero(void* p, size_t bytes) override {
    memset(p, 0, bytes);
    return HEAP_OK;
  }

  int finalize() override {
    if (window_base_) munmap(window_base_, stride_ * npes_);
    window_base_ = nullptr;
    for (int fd : fds_)
      if (fd >= 0) ::close(fd);
    fds_.clear();
    fd_ = -1;
    backed_ = 0;
    return HEAP_OK;
  }

 private:
  std::string name(int pe) const {
    char buf[96];
    snprintf(buf, sizeof(buf), "/bshmem-%016llx-%d", (unsigned long long)key_, pe);
    return buf;
  }
  uint64_t key_ = 0;
  int fd_ = -1;
  std::vector<int> fds_;
};

}  // namespace

std::unique_ptr<SymmetricHeap> make_host_heap() { return std::unique_ptr<SymmetricHeap>(new HostHeap()); }

}  // namespace bshmem
