// Transport plugin loading and the built-in P2P transport (see transport.h).
#include "transport.h"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <string.h>

#include "../state/runtime.h"
#include "../util/env.h"
#include "../util/log.h"

namespace bshmem {
namespace {

// P2P: a peer is reachable when it sits on this host and the two GPUs can address each other's memory; native
// atomics need the P2P atomics attribute; two PEs on one GPU reach each other with plain addresses.
int p2p_can_reach_peer(bshmem_transport*, const PeInfo* me, const PeInfo* peer, int my_device, uint32_t* caps) {
  *caps = 0;
  if (peer->host_hash != me->host_hash) return 0;
  const uint32_t full = TRANSPORT_CAP_MAP | TRANSPORT_CAP_GPU_LD | TRANSPORT_CAP_GPU_ST | TRANSPORT_CAP_CPU_WRITE | TRANSPORT_CAP_CPU_READ;
  if (memcmp(peer->uuid, me->uuid, 16) == 0) {
    *caps = full | TRANSPORT_CAP_GPU_ATOMICS | TRANSPORT_CAP_CPU_ATOMICS | TRANSPORT_CAP_SAME_DEVICE;
    return 0;
  }
  if (options().DISABLE_P2P) return 0;
  int peer_dev = -1;
  if (cudaDeviceGetByPCIBusId(&peer_dev, peer->pci_bus_id) != cudaSuccess || peer_dev < 0) {
    (void)cudaGetLastError();
    return 0;
  }
  int can = 0, atom = 0;
  cudaDeviceCanAccessPeer(&can, my_device, peer_dev);
  cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, my_device, peer_dev);
  if (can) *caps = full;
  if (can && atom) *caps |= TRANSPORT_CAP_GPU_ATOMICS | TRANSPORT_CAP_CPU_ATOMICS;
  return 0;
}
int p2p_show_info(bshmem_transport* t, std::string* out) {
  int reached = 0;
  for (uint32_t c : t->cap) reached += c != 0;
  *out = "P2P (GPU load / store / atomics over NVLink, no endpoints, no proxy): reaches " + std::to_string(reached) + " of " + std::to_string(t->cap.size()) + " PEs";
  return 0;
}
int p2p_finalize(bshmem_transport*) { return 0; }

}  // namespace

int transport_p2p_init(bshmem_transport** out) {
  auto* t = new bshmem_transport();
  t->name = "P2P";
  t->attr = TRANSPORT_ATTR_NO_ENDPOINTS | TRANSPORT_ATTR_NO_REGISTRATION | TRANSPORT_ATTR_NO_PROXY;
  t->ops.can_reach_peer = p2p_can_reach_peer;
  t->ops.show_info = p2p_show_info;
  t->ops.finalize = p2p_finalize;
  *out = t;
  return 0;
}

int transport_load_plugin(const std::string& name, bshmem_transport** out) {
  *out = nullptr;
  const std::string file = "libbshmem_transport_" + name + ".so";
  void* h = dlopen(file.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) {
    ERROR_PRINT("remote transport '%s': dlopen(%s) failed: %s", name.c_str(), file.c_str(), dlerror());
    return 1;
  }
  auto init = (bshmem_transport_init_fn)dlsym(h, "bshmem_transport_init");
  if (!init) {
    ERROR_PRINT("remote transport '%s': %s exports no bshmem_transport_init", name.c_str(), file.c_str());
    dlclose(h);
    return 1;
  }
  bshmem_transport* t = nullptr;
  if (init(&t, BSHMEM_TRANSPORT_API_VERSION) != 0 || !t || t->api_version != BSHMEM_TRANSPORT_API_VERSION || !t->ops.can_reach_peer) {
    ERROR_PRINT("remote transport '%s': initialisation failed or the plugin speaks another interface version", name.c_str());
    dlclose(h);
    return 1;
  }
  t->dl_handle = h;
  *out = t;
  return 0;
}

void transport_destroy(bshmem_transport* t) {
  if (!t) return;
  if (t->ops.finalize) t->ops.finalize(t);
  void* h = t->dl_handle;
  if (!h) delete t;  // a plugin owns its own object
  else dlclose(h);
}

}  // namespace bshmem
