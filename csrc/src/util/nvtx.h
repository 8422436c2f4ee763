// NVTX ranges around public host calls, switched on per group with
// NVSHMEM_NVTX (comma list; "off" by default, "common" = init, alloc, launch,
// coll and memorder, "all" = everything).  The ranges live in the NVTX domain
// "NVSHMEM" so that timelines line up with ones taken from NVSHMEM programs
// (reference: src/include/internal/host/nvshmem_nvtx.hpp, src/host/init/init_nvtx.cpp).
#pragma once
#include <cstdint>

namespace bshmem {

enum NvtxGroup : uint32_t {
  NVTX_INIT = 1u << 0,
  NVTX_ALLOC = 1u << 1,
  NVTX_LAUNCH = 1u << 2,
  NVTX_COLL = 1u << 3,
  NVTX_WAIT = 1u << 4,
  NVTX_WAIT_ON_STREAM = 1u << 5,
  NVTX_TEST = 1u << 6,
  NVTX_MEMORDER = 1u << 7,
  NVTX_QUIET_ON_STREAM = 1u << 8,
  NVTX_ATOMIC_FETCH = 1u << 9,
  NVTX_ATOMIC_SET = 1u << 10,
  NVTX_RMA_BLOCKING = 1u << 11,
  NVTX_RMA_NONBLOCKING = 1u << 12,
  NVTX_PROXY = 1u << 13,
};

void nvtx_init();                       // parses NVSHMEM_NVTX
uint32_t nvtx_mask();
uint32_t nvtx_parse(const char* text);  // exposed for tests
void nvtx_push(const char* name);
void nvtx_pop();

class NvtxRange {
 public:
  NvtxRange(uint32_t group, const char* name) : on_((nvtx_mask() & group) != 0) {
    if (on_) nvtx_push(name);
  }
  ~NvtxRange() {
    if (on_) nvtx_pop();
  }

 private:
  bool on_;
};

}  // namespace bshmem
