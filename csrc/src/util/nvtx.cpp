#include "nvtx.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <sstream>
#include <string>

#include "env.h"

namespace bshmem {

static uint32_t g_mask = 0;
static nvtxDomainHandle_t g_domain = nullptr;

uint32_t nvtx_parse(const char* text) {
  std::string s = text ? text : "";
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  static const struct { const char* name; uint32_t bits; } groups[] = {
      {"off", 0},
      {"common", NVTX_INIT | NVTX_ALLOC | NVTX_LAUNCH | NVTX_COLL | NVTX_MEMORDER},
      {"all", 0xffffffffu},
      {"init", NVTX_INIT}, {"alloc", NVTX_ALLOC}, {"launch", NVTX_LAUNCH}, {"coll", NVTX_COLL},
      {"wait", NVTX_WAIT}, {"wait_on_stream", NVTX_WAIT_ON_STREAM}, {"test", NVTX_TEST},
      {"memorder", NVTX_MEMORDER}, {"quiet_on_stream", NVTX_QUIET_ON_STREAM},
      {"atomic_fetch", NVTX_ATOMIC_FETCH}, {"atomic_set", NVTX_ATOMIC_SET}, {"atomic", NVTX_ATOMIC_FETCH | NVTX_ATOMIC_SET},
      {"rma_blocking", NVTX_RMA_BLOCKING}, {"rma_nonblocking", NVTX_RMA_NONBLOCKING},
      {"rma", NVTX_RMA_BLOCKING | NVTX_RMA_NONBLOCKING}, {"proxy", NVTX_PROXY}};
  uint32_t mask = 0;
  std::stringstream ss(s);
  std::string tok;
  while (std::getline(ss, tok, ','))
    for (auto& g : groups)
      if (tok == g.name) mask |= g.bits;
  return mask;
}

void nvtx_init() {
  g_mask = nvtx_parse(options().NVTX.c_str());
  if (g_mask && !g_domain) g_domain = nvtxDomainCreateA("NVSHMEM");
}

uint32_t nvtx_mask() { return g_mask; }

void nvtx_push(const char* name) {
  nvtxEventAttributes_t a{};
  a.version = NVTX_VERSION;
  a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  a.messageType = NVTX_MESSAGE_TYPE_ASCII;
  a.message.ascii = name;
  nvtxDomainRangePushEx(g_domain, &a);
}

void nvtx_pop() { nvtxDomainRangePop(g_domain); }

}  // namespace bshmem
