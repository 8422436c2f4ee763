// Transport seam of the host library: every way of reaching a peer PE is described by one `bshmem_transport` with a
// table of host operations and, per PE, a set of capability bits.  Bring-up asks each transport which peers it can
// reach and with which capabilities, records the first transport that reaches a peer, and refuses jobs in which some
// peer is reached by none.
//
// One transport is built in: P2P (peers on the same NVLink / NVSwitch domain, reached by loads, stores and atomics
// of the GPU itself, so it needs no endpoints, no memory registration and no proxy).  Further transports are shared
// objects named libbshmem_transport_<name>.so that export `bshmem_transport_init`; NVSHMEM_REMOTE_TRANSPORT=<name>
// loads one at start-up.  None is shipped: network transports are outside what this library targets, the seam is
// what keeps them addable without touching bring-up.
// (reference: src/include/internal/host_transport/transport.h, struct nvshmem_transport and its capability bits;
//  src/host/transport/transport.cpp, src/host/transport/p2p/p2p.cpp)
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace bshmem {

struct PeInfo;

enum TransportCap : uint32_t {
  TRANSPORT_CAP_MAP = 1u << 0,              // the peer's heap can be mapped into this process
  TRANSPORT_CAP_GPU_LD = 1u << 1,           // GPU threads can load from the peer
  TRANSPORT_CAP_GPU_ST = 1u << 2,           // GPU threads can store to the peer
  TRANSPORT_CAP_GPU_ATOMICS = 1u << 3,      // GPU threads can run native atomics on the peer
  TRANSPORT_CAP_CPU_WRITE = 1u << 4,        // host-initiated writes (copy engines or the transport's own path)
  TRANSPORT_CAP_CPU_READ = 1u << 5,
  TRANSPORT_CAP_CPU_ATOMICS = 1u << 6,
  TRANSPORT_CAP_SAME_DEVICE = 1u << 7,      // the peer is another PE on this GPU
};

enum TransportAttr : uint32_t {
  TRANSPORT_ATTR_NO_ENDPOINTS = 1u << 0,    // nothing to connect per peer
  TRANSPORT_ATTR_NO_REGISTRATION = 1u << 1, // local buffers need no registration
  TRANSPORT_ATTR_NO_PROXY = 1u << 2,        // device-initiated operations need no CPU thread
};

struct bshmem_transport;

struct bshmem_transport_host_ops {
  // Capabilities (TransportCap bits) with which this transport reaches `peer`; 0 = cannot reach.
  int (*can_reach_peer)(bshmem_transport* t, const PeInfo* me, const PeInfo* peer, int my_device, uint32_t* caps);
  // Per-peer connection set-up / tear-down for transports with endpoints (null with TRANSPORT_ATTR_NO_ENDPOINTS).
  int (*connect_endpoints)(bshmem_transport* t, const int* pes, int npes);
  // Registration of a range of the symmetric heap (null with TRANSPORT_ATTR_NO_REGISTRATION).
  int (*get_mem_handle)(bshmem_transport* t, void* base, size_t bytes, void* handle_out, size_t handle_bytes);
  int (*release_mem_handle)(bshmem_transport* t, void* handle);
  // Host-initiated data path of transports that carry it themselves (null: copy engines / mapped memory are used).
  int (*rma)(bshmem_transport* t, int pe, void* remote, void* local, size_t bytes, int is_put);
  int (*amo)(bshmem_transport* t, int pe, void* remote, uint64_t value, uint64_t compare, int op, int bytes, uint64_t* fetched);
  int (*quiet)(bshmem_transport* t, int pe);
  int (*fence)(bshmem_transport* t, int pe);
  int (*show_info)(bshmem_transport* t, std::string* out);
  int (*finalize)(bshmem_transport* t);
};

constexpr int BSHMEM_TRANSPORT_API_VERSION = 1;

struct bshmem_transport {
  int api_version = BSHMEM_TRANSPORT_API_VERSION;
  const char* name = "";
  uint32_t attr = 0;
  bshmem_transport_host_ops ops{};
  std::vector<uint32_t> cap;   // per PE, filled at bring-up
  void* state = nullptr;       // the transport's own data
  void* dl_handle = nullptr;   // shared object it came from (null for the built-in one)
};

// Entry point a transport plugin exports (extern "C").
typedef int (*bshmem_transport_init_fn)(bshmem_transport** out, int api_version);

// The built-in load/store transport.
int transport_p2p_init(bshmem_transport** out);
// Loads libbshmem_transport_<name>.so (searched like any shared object) and calls its init.
int transport_load_plugin(const std::string& name, bshmem_transport** out);
void transport_destroy(bshmem_transport* t);

}  // namespace bshmem
