// PMI-1 ("simple PMI") and PMI-2 client bootstrap: lets programs be started by a process manager that speaks the
// PMI wire protocols (Hydra's mpiexec / nvshmrun, Slurm's srun --mpi=pmi / pmi2, or baseline/pmi_launcher.py).
// The manager hands each process a connected socket in PMI_FD plus PMI_RANK and PMI_SIZE.
//   PMI-1: a line protocol of "cmd=... key=value ..." requests and replies (init, get_maxes, get_my_kvsname, put,
//          get, barrier_in, finalize).
//   PMI-2 (NVSHMEM_BOOTSTRAP_PMI=PMI-2): the version is negotiated with one PMI-1 style line, after which every
//          message is a 6-digit decimal length followed by "cmd=...;key=value;..." (fullinit, kvs-put, kvs-fence,
//          kvs-get, finalize, abort).
// Collectives are built from the key-value space in both: every rank puts hex-encoded pieces under keys that carry a
// call sequence number, all ranks pass the manager's barrier (PMI-1) or fence (PMI-2), then read the others' keys.
// (reference: src/modules/bootstrap/pmi/bootstrap_pmi.cpp with its vendored simple-pmi and pmi-2 clients; this file
//  implements both protocols directly instead of vendoring a client.)
#include <ctype.h>
#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../util/env.h"
#include "../util/log.h"
#include "bootstrap.h"

namespace bshmem {
namespace {

struct PmiState {
  int fd = -1;
  int rank = 0, size = 1;
  std::string kvs;
  std::string inbuf;
  uint64_t seq = 0;
  int timeout_ms = 30000;
  bool v2 = false;     // PMI-2 framing and commands
  std::string jobid;   // PMI-2: job id of the key-value space
  size_t piece = 448;  // payload bytes per value: 896 hex characters, inside the usual 1024-character limit
};

bool send_line(PmiState* s, const std::string& line) {
  size_t off = 0;
  while (off < line.size()) {
    ssize_t n = ::write(s->fd, line.data() + off, line.size() - off);
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return false;
    }
    off += (size_t)n;
  }
  return true;
}

// Reads one '\n'-terminated line; false on time-out or a closed socket.
bool recv_line(PmiState* s, std::string* out) {
  for (;;) {
    size_t nl = s->inbuf.find('\n');
    if (nl != std::string::npos) {
      *out = s->inbuf.substr(0, nl);
      s->inbuf.erase(0, nl + 1);
      return true;
    }
    struct pollfd p = {s->fd, POLLIN, 0};
    int r = ::poll(&p, 1, s->timeout_ms);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    char buf[4096];
    ssize_t n = ::read(s->fd, buf, sizeof(buf));
    if (n == 0) return false;
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return false;
    }
    s->inbuf.append(buf, (size_t)n);
  }
}

// Value of `key` in a reply line of space-separated key=value tokens ("" if absent).
std::string field(const std::string& line, const char* key) {
  const std::string pat = std::string(key) + "=";
  size_t pos = 0;
  while (pos < line.size()) {
    size_t end = line.find(' ', pos);
    if (end == std::string::npos) end = line.size();
    if (line.compare(pos, pat.size(), pat) == 0) return line.substr(pos + pat.size(), end - pos - pat.size());
    pos = end + 1;
  }
  return "";
}

int request(PmiState* s, const std::string& req, const char* want_cmd, std::string* reply) {
  if (!send_line(s, req)) return BOOT_ERR_SOCKET;
  std::string line;
  if (!recv_line(s, &line)) return BOOT_ERR_TIMEOUT;
  if (field(line, "cmd") != want_cmd) {
    ERROR_PRINT("PMI: expected '%s', got '%s'", want_cmd, line.c_str());
    return BOOT_ERR_PEER;
  }
  if (reply) *reply = line;
  return BOOT_OK;
}

// ---- PMI-2 framing: "%6u" length, then a body of ';'-terminated key=value pairs
bool send_v2(PmiState* s, const std::string& body) {
  char len[8];
  snprintf(len, sizeof(len), "%6u", (unsigned)body.size());
  return send_line(s, std::string(len, 6) + body);
}
bool recv_v2(PmiState* s, std::string* body) {
  auto fill = [&](size_t want) {
    while (s->inbuf.size() < want) {
      struct pollfd p = {s->fd, POLLIN, 0};
      int r = ::poll(&p, 1, s->timeout_ms);
      if (r == 0) return false;
      if (r < 0) {
        if (errno == EINTR) continue;
        return false;
      }
      char buf[4096];
      ssize_t n = ::read(s->fd, buf, sizeof(buf));
      if (n == 0) return false;
      if (n < 0) {
        if (errno == EINTR || errno == EAGAIN) continue;
        return false;
      }
      s->inbuf.append(buf, (size_t)n);
    }
    return true;
  };
  if (!fill(6)) return false;
  const size_t len = (size_t)strtoul(s->inbuf.substr(0, 6).c_str(), nullptr, 10);
  if (len == 0 || len > (1u << 20) || !fill(6 + len)) return false;
  *body = s->inbuf.substr(6, len);
  s->inbuf.erase(0, 6 + len);
  return true;
}
std::string field_v2(const std::string& body, const char* key) {
  const std::string pat = std::string(key) + "=";
  size_t pos = 0;
  while (pos < body.size()) {
    size_t end = body.find(';', pos);
    if (end == std::string::npos) end = body.size();
    if (body.compare(pos, pat.size(), pat) == 0) return body.substr(pos + pat.size(), end - pos - pat.size());
    pos = end + 1;
  }
  return "";
}
int request_v2(PmiState* s, const std::string& body, const char* want_cmd, std::string* reply) {
  if (!send_v2(s, body)) return BOOT_ERR_SOCKET;
  std::string r;
  if (!recv_v2(s, &r)) return BOOT_ERR_TIMEOUT;
  if (field_v2(r, "cmd") != want_cmd || field_v2(r, "rc") != "0") {
    ERROR_PRINT("PMI-2: expected '%s' with rc=0, got '%s'", want_cmd, r.c_str());
    return BOOT_ERR_PEER;
  }
  if (reply) *reply = r;
  return BOOT_OK;
}

std::string to_hex(const unsigned char* p, size_t n) {
  static const char d[] = "0123456789abcdef";
  std::string out(2 * n, '0');
  for (size_t i = 0; i < n; ++i) {
    out[2 * i] = d[p[i] >> 4];
    out[2 * i + 1] = d[p[i] & 15];
  }
  return out;
}
bool from_hex(const std::string& h, unsigned char* p, size_t n) {
  if (h.size() != 2 * n) return false;
  auto v = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : -1; };
  for (size_t i = 0; i < n; ++i) {
    int a = v(h[2 * i]), b = v(h[2 * i + 1]);
    if (a < 0 || b < 0) return false;
    p[i] = (unsigned char)(a * 16 + b);
  }
  return true;
}

int kvs_put(PmiState* s, const std::string& key, const unsigned char* data, size_t n) {
  for (size_t off = 0, part = 0; off < n || (n == 0 && part == 0); off += s->piece, ++part) {
    size_t len = n - off < s->piece ? n - off : s->piece;
    std::string reply;
    if (s->v2) {
      int st2 = request_v2(s, "cmd=kvs-put;key=" + key + "." + std::to_string(part) + ";value=" + to_hex(data + off, len) + ";", "kvs-put-response", nullptr);
      if (st2 != BOOT_OK) return st2;
      if (n == 0) break;
      continue;
    }
    int st = request(s, "cmd=put kvsname=" + s->kvs + " key=" + key + "." + std::to_string(part) + " value=" + to_hex(data + off, len) + "\n", "put_result", &reply);
    if (st != BOOT_OK) return st;
    if (field(reply, "rc") != "0") return BOOT_ERR_PEER;
    if (n == 0) break;
  }
  return BOOT_OK;
}
int kvs_get(PmiState* s, const std::string& key, unsigned char* data, size_t n) {
  for (size_t off = 0, part = 0; off < n; off += s->piece, ++part) {
    size_t len = n - off < s->piece ? n - off : s->piece;
    std::string reply;
    if (s->v2) {
      int st2 = request_v2(s, "cmd=kvs-get;jobid=" + s->jobid + ";srcid=-1;key=" + key + "." + std::to_string(part) + ";", "kvs-get-response", &reply);
      if (st2 != BOOT_OK) return st2;
      if (field_v2(reply, "found") != "TRUE" || !from_hex(field_v2(reply, "value"), data + off, len)) {
        ERROR_PRINT("PMI-2: key %s.%zu is missing or malformed", key.c_str(), part);
        return BOOT_ERR_PEER;
      }
      continue;
    }
    int st = request(s, "cmd=get kvsname=" + s->kvs + " key=" + key + "." + std::to_string(part) + "\n", "get_result", &reply);
    if (st != BOOT_OK) return st;
    if (field(reply, "rc") != "0" || !from_hex(field(reply, "value"), data + off, len)) {
      ERROR_PRINT("PMI: key %s.%zu is missing or malformed", key.c_str(), part);
      return BOOT_ERR_PEER;
    }
  }
  return BOOT_OK;
}

int pmi_barrier(bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  if (s->size == 1) return BOOT_OK;
  if (s->v2) return request_v2(s, "cmd=kvs-fence;", "kvs-fence-response", nullptr);
  return request(s, "cmd=barrier_in\n", "barrier_out", nullptr);
}

int pmi_allgather(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  const uint64_t seq = s->seq++;
  memcpy((char*)recvbuf + (size_t)s->rank * bytes, sendbuf, (size_t)bytes);
  if (s->size == 1) return BOOT_OK;
  int st = kvs_put(s, "ag" + std::to_string(seq) + "-" + std::to_string(s->rank), (const unsigned char*)sendbuf, (size_t)bytes);
  if (st == BOOT_OK) st = pmi_barrier(h);
  for (int r = 0; r < s->size && st == BOOT_OK; ++r)
    if (r != s->rank) st = kvs_get(s, "ag" + std::to_string(seq) + "-" + std::to_string(r), (unsigned char*)recvbuf + (size_t)r * bytes, (size_t)bytes);
  return st;
}

int pmi_alltoall(const void* sendbuf, void* recvbuf, int bytes, bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  const uint64_t seq = s->seq++;
  memcpy((char*)recvbuf + (size_t)s->rank * bytes, (const char*)sendbuf + (size_t)s->rank * bytes, (size_t)bytes);
  if (s->size == 1) return BOOT_OK;
  int st = BOOT_OK;
  for (int r = 0; r < s->size && st == BOOT_OK; ++r)
    if (r != s->rank)
      st = kvs_put(s, "aa" + std::to_string(seq) + "-" + std::to_string(s->rank) + "-" + std::to_string(r), (const unsigned char*)sendbuf + (size_t)r * bytes, (size_t)bytes);
  if (st == BOOT_OK) st = pmi_barrier(h);
  for (int r = 0; r < s->size && st == BOOT_OK; ++r)
    if (r != s->rank)
      st = kvs_get(s, "aa" + std::to_string(seq) + "-" + std::to_string(r) + "-" + std::to_string(s->rank), (unsigned char*)recvbuf + (size_t)r * bytes, (size_t)bytes);
  return st;
}

void pmi_global_exit(int status, bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  if (s && s->fd >= 0) {
    if (s->v2) send_v2(s, "cmd=abort;isworld=TRUE;msg=global_exit;exitcode=" + std::to_string(status) + ";");
    else send_line(s, "cmd=abort exitcode=" + std::to_string(status) + "\n");
  }
  _exit(status);
}

int pmi_finalize(bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  if (!s) return BOOT_OK;
  if (s->fd >= 0) {
    if (s->v2) request_v2(s, "cmd=finalize;", "finalize-response", nullptr);
    else request(s, "cmd=finalize\n", "finalize_ack", nullptr);
  }
  delete s;
  h->comm_state = nullptr;
  return BOOT_OK;
}

int pmi_show_info(bshmem_bootstrap_handle_t* h) {
  PmiState* s = (PmiState*)h->comm_state;
  INFO(SUB_BOOTSTRAP, "%s bootstrap: rank %d of %d, key-value space '%s'", s->v2 ? "PMI-2" : "PMI-1", s->rank, s->size, s->v2 ? s->jobid.c_str() : s->kvs.c_str());
  return BOOT_OK;
}

}  // namespace

bool bootstrap_pmi_available() { return getenv("PMI_FD") && getenv("PMI_RANK") && getenv("PMI_SIZE"); }

int bootstrap_pmi_init(bshmem_bootstrap_handle_t* handle) {
  if (!bootstrap_pmi_available()) {
    ERROR_PRINT("PMI bootstrap: PMI_FD, PMI_RANK and PMI_SIZE are not set (start the program under a PMI process manager)");
    return BOOT_ERR_ARGS;
  }
  PmiState* s = new PmiState;
  s->fd = atoi(getenv("PMI_FD"));
  s->rank = atoi(getenv("PMI_RANK"));
  s->size = atoi(getenv("PMI_SIZE"));
  s->timeout_ms = (int)options().BOOTSTRAP_TIMEOUT_MS > 0 ? (int)options().BOOTSTRAP_TIMEOUT_MS : 30000;
  std::string reply;
  std::string want = options().BOOTSTRAP_PMI;
  for (auto& c : want) c = (char)toupper(c);
  s->v2 = want == "PMI-2" || want == "PMI2";
  int st;
  if (s->v2) {
    // The version is agreed with one PMI-1 style line; everything after it is length-prefixed.
    st = request(s, "cmd=init pmi_version=2 pmi_subversion=0\n", "response_to_init", &reply);
    if (st == BOOT_OK && (field(reply, "rc") != "0" || field(reply, "pmi_version") != "2")) st = BOOT_ERR_VERSION;
    const char* jid = getenv("PMI_JOBID");
    if (st == BOOT_OK)
      st = request_v2(s, std::string("cmd=fullinit;pmijobid=") + (jid ? jid : "0") + ";pmirank=" + std::to_string(s->rank) + ";threaded=FALSE;", "fullinit-response", &reply);
    if (st == BOOT_OK) {
      s->rank = atoi(field_v2(reply, "rank").c_str());
      s->size = atoi(field_v2(reply, "size").c_str());
      st = request_v2(s, "cmd=job-getid;", "job-getid-response", &reply);
    }
    if (st == BOOT_OK) s->jobid = field_v2(reply, "jobid");
    s->kvs = s->jobid;
  } else {
    st = request(s, "cmd=init pmi_version=1 pmi_subversion=1\n", "response_to_init", &reply);
    if (st == BOOT_OK && field(reply, "rc") != "0") st = BOOT_ERR_VERSION;
    if (st == BOOT_OK) st = request(s, "cmd=get_maxes\n", "maxes", &reply);
    if (st == BOOT_OK) {
      const long vallen = atol(field(reply, "vallen_max").c_str());
      if (vallen >= 64) s->piece = (size_t)((vallen - 2) / 2) < s->piece ? (size_t)((vallen - 2) / 2) : s->piece;
      st = request(s, "cmd=get_my_kvsname\n", "my_kvsname", &reply);
    }
    if (st == BOOT_OK) s->kvs = field(reply, "kvsname");
  }
  if (st != BOOT_OK || s->kvs.empty() || s->rank < 0 || s->rank >= s->size) {
    ERROR_PRINT("PMI bootstrap: handshake with the process manager failed (%s)", bootstrap_strerror(st));
    delete s;
    return st != BOOT_OK ? st : BOOT_ERR_PEER;
  }
  handle->version = BSHMEM_BOOTSTRAP_ABI_VERSION;
  handle->pg_rank = s->rank;
  handle->pg_size = s->size;
  handle->allgather = pmi_allgather;
  handle->alltoall = pmi_alltoall;
  handle->barrier = pmi_barrier;
  handle->global_exit = pmi_global_exit;
  handle->finalize = pmi_finalize;
  handle->show_info = pmi_show_info;
  handle->comm_state = s;
  return BOOT_OK;
}

}  // namespace bshmem
