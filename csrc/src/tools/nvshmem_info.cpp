// nvshmem-info: prints the library version (-n), the build options (-b), the environment variables
// with their current values (-e; -d adds hidden ones, -r prints reStructuredText), or everything (-a)
// (reference: src/bin/nvshmem-info.cpp).
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include "../../include/bshmem/state.h"
#include "../util/env.h"

using namespace bshmem;

static void usage(const char* argv0) {
  printf("usage: %s [-a] [-n] [-b] [-e] [-d] [-r] [-h]\n"
         "  -n  version\n  -b  build options\n  -e  environment variables\n  -d  include hidden variables\n  -r  reStructuredText output\n  -a  all of the above\n",
         argv0);
}

static const char* cat_name(OptCat c) {
  switch (c) {
    case OptCat::OpenShmem: return "Standard options";
    case OptCat::Bootstrap: return "Bootstrap options";
    case OptCat::Collectives: return "Collectives options";
    case OptCat::Memory: return "Memory options";
    case OptCat::Transport: return "Transport options";
    case OptCat::Debug: return "Debugging options";
    case OptCat::Accepted: return "Options of the reference that are accepted and change nothing here";
    default: return "Hidden options";
  }
}

int main(int argc, char** argv) {
  bool version = false, build = false, env = false, hidden = false, rst = false;
  int c;
  if (argc == 1) version = true;
  while ((c = getopt(argc, argv, "anbedrh")) != -1) {
    switch (c) {
      case 'a': version = build = env = true; break;
      case 'n': version = true; break;
      case 'b': build = true; break;
      case 'e': env = true; break;
      case 'd': env = hidden = true; break;
      case 'r': rst = true; break;
      default: usage(argv[0]); return c == 'h' ? 0 : 1;
    }
  }
  if (version) printf("%s v%d.%d.%d (OpenSHMEM %d.%d semantics)\n", BSHMEM_VENDOR_STRING, BSHMEM_MAJOR, BSHMEM_MINOR, BSHMEM_PATCH, 1, 3);
  if (build) {
    printf("Build information:\n");
    printf("  %-36s %s\n", "CUDA architectures", "sm_100a");
    printf("  %-36s %s\n", "Bootstraps", "UID (built in), plugin loader");
    printf("  %-36s %s\n", "Transports", "NVLink load/store, NVLS multicast");
    printf("  %-36s %s\n", "Remote transports (IB, UCX, OFI)", "none shipped; plugin seam libbshmem_transport_<name>.so (NVSHMEM_REMOTE_TRANSPORT)");
    printf("  %-36s %s\n", "Heap back ends", "CUDA VMM, host shared memory");
    printf("  %-36s %s\n", "Device waits", "bounded (NVSHMEM_WAIT_TIMEOUT_MS)");
    printf("  %-36s %d\n", "Maximum PEs for stack arrays", BSHMEM_MAX_PES);
    printf("  %-36s %d\n", "Barrier rows per team", BSHMEM_SYNC_SLOTS);
  }
  if (env) {
    Options o;
    options_init(&o);
    OptCat last = (OptCat)-1;
    for (auto& i : options_describe(o)) {
      if (i.cat == OptCat::Hidden && !hidden) continue;
      if (i.cat != last) {
        last = i.cat;
        if (rst) printf("\n%s\n%s\n\n", cat_name(i.cat), std::string(strlen(cat_name(i.cat)), '~').c_str());
        else printf("\n%s:\n", cat_name(i.cat));
      }
      if (rst) printf(".. c:var:: %s\n\n   Default: %s\n\n   %s\n\n", i.name, i.dflt.c_str(), i.help);
      else printf("  %-40s %s (default %s)%s\n      %s\n", i.name, i.value.c_str(), i.dflt.c_str(), i.set ? " [set]" : "", i.help);
    }
  }
  return 0;
}
