#include "cuda_dl.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "log.h"

namespace bshmem {

#define BSHMEM_STR2(x) #x
#define BSHMEM_STR(x) BSHMEM_STR2(x)

static CuTable g_tab;
static bool g_ok = false;
static std::string g_missing;
static std::once_flag g_once;

const CuTable* cu(std::string* missing) {
  std::call_once(g_once, [] {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      g_missing = "libcuda.so.1";
      return;
    }
    // cuda.h maps the plain names to versioned symbols with macros; stringifying
    // the macro-expanded token gives the symbol that the header's prototype describes.
#define X(name)                                                      \
  g_tab.name##_ = (decltype(g_tab.name##_))dlsym(lib, BSHMEM_STR(name)); \
  if (!g_tab.name##_) { g_missing += BSHMEM_STR(name); g_missing += " "; }
    BSHMEM_CU_FUNCS(X)
#undef X
    g_ok = g_tab.cuInit_ != nullptr;
  });
  if (missing) *missing = g_missing;
  return g_ok ? &g_tab : nullptr;
}

std::string cu_error_string(CUresult r) {
  const CuTable* t = cu();
  const char* s = nullptr;
  if (t && t->cuGetErrorString_ && t->cuGetErrorString_(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUresult " + std::to_string((int)r);
}

// ---------------------------------------------------------------- NVML
// Only a handful of calls, declared locally so that nvml.h is not needed.
namespace {
typedef void* nvmlDevice_t;
typedef int (*nvmlInit_t)();
typedef int (*nvmlShutdown_t)();
typedef int (*nvmlGetHandleByPci_t)(const char*, nvmlDevice_t*);
typedef int (*nvmlGetNvLinkState_t)(nvmlDevice_t, unsigned, int*);
typedef int (*nvmlGetNvLinkVersion_t)(nvmlDevice_t, unsigned, unsigned*);
typedef int (*nvmlGetDriverVersion_t)(char*, unsigned);
struct NvmlPciInfo {  // nvmlPciInfo_t, v2 layout
  char busIdLegacy[16];
  unsigned domain, bus, device, pciDeviceId, pciSubSystemId;
  char busId[32];
};
typedef int (*nvmlGetNvLinkRemotePci_t)(nvmlDevice_t, unsigned, NvmlPciInfo*);
}  // namespace

NvlinkInfo nvml_probe_nvlink(const char* pci_bus_id) {
  NvlinkInfo info;
  void* lib = dlopen("libnvidia-ml.so.1", RTLD_NOW);
  if (!lib) return info;
  auto init = (nvmlInit_t)dlsym(lib, "nvmlInit_v2");
  auto shut = (nvmlShutdown_t)dlsym(lib, "nvmlShutdown");
  auto by_pci = (nvmlGetHandleByPci_t)dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2");
  auto state = (nvmlGetNvLinkState_t)dlsym(lib, "nvmlDeviceGetNvLinkState");
  auto version = (nvmlGetNvLinkVersion_t)dlsym(lib, "nvmlDeviceGetNvLinkVersion");
  auto drv = (nvmlGetDriverVersion_t)dlsym(lib, "nvmlSystemGetDriverVersion");
  if (!init || !shut || !by_pci || !state || init() != 0) {
    dlclose(lib);
    return info;
  }
  info.nvml_loaded = true;
  char ver[96] = "";
  if (drv && drv(ver, sizeof(ver)) == 0) info.driver_version = ver;
  nvmlDevice_t dev = nullptr;
  if (by_pci(pci_bus_id, &dev) == 0) {
    for (unsigned link = 0; link < 18; ++link) {  // NVLink 5: up to 18 links per GPU
      int active = 0;
      if (state(dev, link, &active) != 0) break;
      if (!active) continue;
      ++info.active_links;
      unsigned v = 0;
      if (version && version(dev, link, &v) == 0) info.link_version = (int)v;
    }
    // On an NVSwitch box every link of every GPU ends in a switch, so all
    // peers are equally near; a full set of active links is the sign looked for.
    info.all_links_to_switch = info.active_links >= 18;
  }
  shut();
  dlclose(lib);
  return info;
}

}  // namespace bshmem
