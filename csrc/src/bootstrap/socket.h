// Small TCP layer for the out-of-band bootstrap: listen/connect/accept with a
// magic handshake, full-length send/recv and a deadlock-free simultaneous
// exchange, every call bounded by a deadline and returning a status instead of
// exiting.  Also picks the network interface (NVSHMEM_BOOTSTRAP_UID_SOCK_IFNAME
// and _FAMILY), falling back to loopback so that a single box with an
// unresolvable host name still works
// (reference: src/modules/bootstrap/uid/ncclSocket/ncclsocket_socket.cpp).
#pragma once
#include <netinet/in.h>
#include <sys/socket.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace bshmem {

enum SockStatus { SOCK_OK = 0, SOCK_TIMEOUT = 1, SOCK_CLOSED = 2, SOCK_ERROR = 3, SOCK_BAD_MAGIC = 4 };
const char* sock_strerror(int st);

// Portable address: fits in the 124 opaque bytes of a unique id.
struct SockAddr {
  uint16_t family;  // AF_INET or AF_INET6
  uint16_t port;    // host byte order
  uint8_t addr[16];
  uint32_t scope_id;
  std::string str() const;
};

// Chooses the address this process listens on.  `ifname_spec` follows the
// NVSHMEM/NCCL convention: "eth" prefix match, "=eth0" exact, "^lo,docker"
// exclusion; empty = first non-loopback interface that is up, else loopback.
int sock_pick_address(const std::string& ifname_spec, const std::string& family, SockAddr* out, std::string* ifname_out = nullptr);
bool sock_parse_hostport(const std::string& text, SockAddr* out);  // "127.0.0.1:12345", "[::1]:999"

// Listening socket bound to `addr` (port 0 = ephemeral; the chosen port is written back).
int sock_listen(SockAddr* addr, int* fd_out, int backlog = 1024);
// Connect, retrying on ECONNREFUSED until the deadline; sends `magic` first.
int sock_connect(const SockAddr& addr, uint64_t magic, int timeout_ms, int* fd_out, const volatile int* abort_flag = nullptr);
// Accept one connection and check its magic.  A connection with the wrong
// magic is closed and reported as SOCK_BAD_MAGIC (the caller usually retries).
int sock_accept(int listen_fd, uint64_t magic, int timeout_ms, int* fd_out, const volatile int* abort_flag = nullptr);

int sock_send(int fd, const void* buf, size_t len, int timeout_ms);
int sock_recv(int fd, void* buf, size_t len, int timeout_ms);
// Sends on one socket and receives on another at the same time (either may be
// the same fd), so that ring and pairwise patterns cannot deadlock on full buffers.
int sock_exchange(int send_fd, const void* sbuf, size_t slen, int recv_fd, void* rbuf, size_t rlen, int timeout_ms);
void sock_close(int fd);

}  // namespace bshmem
