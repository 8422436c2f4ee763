#include "socket.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <sstream>
#include <vector>

#include "../util/log.h"

namespace bshmem {

const char* sock_strerror(int st) {
  switch (st) {
    case SOCK_OK: return "ok";
    case SOCK_TIMEOUT: return "timed out";
    case SOCK_CLOSED: return "connection closed by peer";
    case SOCK_BAD_MAGIC: return "handshake magic mismatch";
    default: return "socket error";
  }
}

static int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

std::string SockAddr::str() const {
  char buf[INET6_ADDRSTRLEN] = "";
  inet_ntop(family, addr, buf, sizeof(buf));
  std::ostringstream os;
  if (family == AF_INET6) os << "[" << buf << "]:" << port;
  else os << buf << ":" << port;
  return os.str();
}

static socklen_t to_sockaddr(const SockAddr& a, sockaddr_storage* ss) {
  memset(ss, 0, sizeof(*ss));
  if (a.family == AF_INET6) {
    auto* s6 = (sockaddr_in6*)ss;
    s6->sin6_family = AF_INET6;
    s6->sin6_port = htons(a.port);
    memcpy(&s6->sin6_addr, a.addr, 16);
    s6->sin6_scope_id = a.scope_id;
    return sizeof(sockaddr_in6);
  }
  auto* s4 = (sockaddr_in*)ss;
  s4->sin_family = AF_INET;
  s4->sin_port = htons(a.port);
  memcpy(&s4->sin_addr, a.addr, 4);
  return sizeof(sockaddr_in);
}

static void from_sockaddr(const sockaddr* sa, SockAddr* out) {
  memset(out, 0, sizeof(SockAddr) - sizeof(uint32_t));
  out->scope_id = 0;
  if (sa->sa_family == AF_INET6) {
    auto* s6 = (const sockaddr_in6*)sa;
    out->family = AF_INET6;
    out->port = ntohs(s6->sin6_port);
    memcpy(out->addr, &s6->sin6_addr, 16);
    out->scope_id = s6->sin6_scope_id;
  } else {
    auto* s4 = (const sockaddr_in*)sa;
    out->family = AF_INET;
    out->port = ntohs(s4->sin_port);
    memcpy(out->addr, &s4->sin_addr, 4);
  }
}

static bool ifname_matches(const std::string& spec, const char* name, bool* is_exclusion) {
  // spec: "", "eth,ib", "=eth0", "^lo,docker"
  *is_exclusion = false;
  if (spec.empty()) return true;
  std::string s = spec;
  bool exact = false;
  if (s[0] == '^') { *is_exclusion = true; s = s.substr(1); }
  else if (s[0] == '=') { exact = true; s = s.substr(1); }
  std::stringstream ss(s);
  std::string tok;
  bool hit = false;
  while (std::getline(ss, tok, ',')) {
    if (tok.empty()) continue;
    if (exact ? tok == name : strncmp(name, tok.c_str(), tok.size()) == 0) hit = true;
  }
  return *is_exclusion ? !hit : hit;
}

int sock_pick_address(const std::string& ifname_spec, const std::string& family, SockAddr* out, std::string* ifname_out) {
  int want = (family == "AF_INET6") ? AF_INET6 : AF_INET;
  ifaddrs* list = nullptr;
  SockAddr loop{};
  bool have_loop = false, found = false;
  std::string loop_name;
  if (getifaddrs(&list) == 0) {
    for (ifaddrs* it = list; it && !found; it = it->ifa_next) {
      if (!it->ifa_addr || it->ifa_addr->sa_family != want) continue;
      if (!(it->ifa_flags & IFF_UP)) continue;
      bool excl;
      if (!ifname_matches(ifname_spec, it->ifa_name, &excl)) continue;
      if (it->ifa_flags & IFF_LOOPBACK) {
        if (!have_loop) { from_sockaddr(it->ifa_addr, &loop); have_loop = true; loop_name = it->ifa_name; }
        // An explicit (non-exclusion) request for the loopback interface is honoured at once.
        if (!ifname_spec.empty() && !excl) { *out = loop; found = true; if (ifname_out) *ifname_out = it->ifa_name; }
        continue;
      }
      from_sockaddr(it->ifa_addr, out);
      if (ifname_out) *ifname_out = it->ifa_name;
      found = true;
    }
    freeifaddrs(list);
  }
  if (!found) {
    if (have_loop) {
      *out = loop;
      if (ifname_out) *ifname_out = loop_name;
    } else {
      memset(out, 0, sizeof(*out));
      out->family = (uint16_t)want;
      if (want == AF_INET) { out->addr[0] = 127; out->addr[3] = 1; } else { out->addr[15] = 1; }
      if (ifname_out) *ifname_out = "lo";
    }
  }
  out->port = 0;
  return SOCK_OK;
}

bool sock_parse_hostport(const std::string& text, SockAddr* out) {
  memset(out, 0, sizeof(*out));
  std::string host, port;
  if (!text.empty() && text[0] == '[') {
    size_t rb = text.find(']');
    if (rb == std::string::npos || rb + 2 > text.size() || text[rb + 1] != ':') return false;
    host = text.substr(1, rb - 1);
    port = text.substr(rb + 2);
    out->family = AF_INET6;
    if (inet_pton(AF_INET6, host.c_str(), out->addr) != 1) return false;
  } else {
    size_t c = text.rfind(':');
    if (c == std::string::npos) return false;
    host = text.substr(0, c);
    port = text.substr(c + 1);
    out->family = AF_INET;
    if (inet_pton(AF_INET, host.c_str(), out->addr) != 1) return false;
  }
  char* end = nullptr;
  long p = strtol(port.c_str(), &end, 10);
  if (end == port.c_str() || *end || p <= 0 || p > 65535) return false;
  out->port = (uint16_t)p;
  return true;
}

static void set_nonblock(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}

static void tune(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  set_nonblock(fd, true);
}

int sock_listen(SockAddr* addr, int* fd_out, int backlog) {
  int fd = socket(addr->family, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return SOCK_ERROR;
  int one = 1;
  if (addr->port != 0) setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_storage ss;
  socklen_t len = to_sockaddr(*addr, &ss);
  if (bind(fd, (sockaddr*)&ss, len) != 0 || listen(fd, backlog) != 0) {
    ERROR_PRINT("bootstrap: cannot listen on %s: %s", addr->str().c_str(), strerror(errno));
    close(fd);
    return SOCK_ERROR;
  }
  socklen_t l2 = sizeof(ss);
  getsockname(fd, (sockaddr*)&ss, &l2);
  SockAddr bound;
  from_sockaddr((sockaddr*)&ss, &bound);
  addr->port = bound.port;
  set_nonblock(fd, true);
  *fd_out = fd;
  return SOCK_OK;
}

static int wait_fd(int fd, short events, int64_t deadline, const volatile int* abort_flag) {
  for (;;) {
    int64_t left = deadline - now_ms();
    if (left <= 0) return SOCK_TIMEOUT;
    if (abort_flag && *abort_flag) return SOCK_CLOSED;
    pollfd p{fd, events, 0};
    int r = poll(&p, 1, (int)std::min<int64_t>(left, 100));
    if (r < 0 && errno == EINTR) continue;
    if (r < 0) return SOCK_ERROR;
    if (r > 0) return SOCK_OK;  // readable/writable, or an error the next syscall will report
  }
}

int sock_connect(const SockAddr& addr, uint64_t magic, int timeout_ms, int* fd_out, const volatile int* abort_flag) {
  int64_t deadline = now_ms() + timeout_ms;
  sockaddr_storage ss;
  socklen_t len = to_sockaddr(addr, &ss);
  for (;;) {
    int fd = socket(addr.family, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return SOCK_ERROR;
    tune(fd);
    int r = connect(fd, (sockaddr*)&ss, len);
    int err = r == 0 ? 0 : errno;
    if (err == EINPROGRESS) {
      int w = wait_fd(fd, POLLOUT, deadline, abort_flag);
      if (w != SOCK_OK) { close(fd); return w; }
      socklen_t el = sizeof(err);
      getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el);
    }
    if (err == 0) {
      int st = sock_send(fd, &magic, sizeof(magic), (int)std::max<int64_t>(1, deadline - now_ms()));
      if (st != SOCK_OK) { close(fd); return st; }
      *fd_out = fd;
      return SOCK_OK;
    }
    close(fd);
    if (err != ECONNREFUSED && err != ETIMEDOUT && err != EAGAIN) {
      ERROR_PRINT("bootstrap: connect to %s failed: %s", addr.str().c_str(), strerror(err));
      return SOCK_ERROR;
    }
    if (now_ms() >= deadline) return SOCK_TIMEOUT;
    if (abort_flag && *abort_flag) return SOCK_CLOSED;
    usleep(2000);  // the listener is not up yet
  }
}

int sock_accept(int listen_fd, uint64_t magic, int timeout_ms, int* fd_out, const volatile int* abort_flag) {
  int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    int w = wait_fd(listen_fd, POLLIN, deadline, abort_flag);
    if (w != SOCK_OK) return w;
    int fd = accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR || errno == ECONNABORTED) continue;
      return SOCK_ERROR;
    }
    tune(fd);
    uint64_t got = 0;
    int st = sock_recv(fd, &got, sizeof(got), (int)std::max<int64_t>(1, std::min<int64_t>(deadline - now_ms(), 5000)));
    if (st != SOCK_OK || got != magic) {
      // Not one of ours: wrong number, or a connection that closed or stayed silent before sending one.
      close(fd);
      return SOCK_BAD_MAGIC;
    }
    *fd_out = fd;
    return SOCK_OK;
  }
}

int sock_send(int fd, const void* buf, size_t len, int timeout_ms) {
  return sock_exchange(fd, buf, len, -1, nullptr, 0, timeout_ms);
}

int sock_recv(int fd, void* buf, size_t len, int timeout_ms) {
  return sock_exchange(-1, nullptr, 0, fd, buf, len, timeout_ms);
}

int sock_exchange(int sfd, const void* sbuf, size_t slen, int rfd, void* rbuf, size_t rlen, int timeout_ms) {
  int64_t deadline = now_ms() + timeout_ms;
  size_t sent = 0, got = 0;
  const char* sp = (const char*)sbuf;
  char* rp = (char*)rbuf;
  while (sent < slen || got < rlen) {
    pollfd p[2];
    int n = 0, si = -1, ri = -1;
    if (sent < slen) { p[n] = {sfd, POLLOUT, 0}; si = n++; }
    if (got < rlen) { p[n] = {rfd, POLLIN, 0}; ri = n++; }
    int64_t left = deadline - now_ms();
    if (left <= 0) return SOCK_TIMEOUT;
    int r = poll(p, n, (int)std::min<int64_t>(left, 200));
    if (r < 0 && errno == EINTR) continue;
    if (r < 0) return SOCK_ERROR;
    if (r == 0) continue;
    if (si >= 0 && (p[si].revents & (POLLOUT | POLLERR | POLLHUP))) {
      ssize_t w = ::send(sfd, sp + sent, slen - sent, MSG_NOSIGNAL);
      if (w > 0) sent += (size_t)w;
      else if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)
        return (errno == EPIPE || errno == ECONNRESET) ? SOCK_CLOSED : SOCK_ERROR;
    }
    if (ri >= 0 && (p[ri].revents & (POLLIN | POLLERR | POLLHUP))) {
      ssize_t g = ::recv(rfd, rp + got, rlen - got, 0);
      if (g > 0) got += (size_t)g;
      else if (g == 0) return SOCK_CLOSED;
      else if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)
        return errno == ECONNRESET ? SOCK_CLOSED : SOCK_ERROR;
    }
  }
  return SOCK_OK;
}

void sock_close(int fd) {
  if (fd >= 0) close(fd);
}

}  // namespace bshmem
