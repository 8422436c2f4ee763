// Smallest program: initialise, say who we are, finalise.  Host code only (no CUDA compiler needed).
//   python -m nvshmem_b200.launch -n 2 -- examples/bin/hello
// (counterpart of the reference's examples/hello.cpp)
#include <stdio.h>

#include "nvshmem.h"

int main() {
  nvshmem_init();
  int major = 0, minor = 0;
  char name[NVSHMEM_MAX_NAME_LEN];
  nvshmem_info_get_version(&major, &minor);
  nvshmem_info_get_name(name);
  printf("Hello from PE %d of %d (%s, OpenSHMEM %d.%d)\n", nvshmem_my_pe(), nvshmem_n_pes(), name, major, minor);
  nvshmem_barrier_all();
  nvshmem_finalize();
  return 0;
}
