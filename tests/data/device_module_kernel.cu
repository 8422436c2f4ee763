// Device code that is compiled on its own into a cubin and loaded with the driver API (no host code, no static
// registrar): BSHMEM_DEVICE_MODULE gives the module's copy of the library state the global name that
// nvshmemx_cumodule_init looks up.
#define BSHMEM_DEVICE_MODULE
#include <nvshmem.h>

// One CTA: puts `n` ints into `dst` on PE `pe`, completes them, then raises `sig` there.
extern "C" __global__ void module_put(int* dst, const int* src, int n, uint64_t* sig, int pe, int* facts) {
  nvshmemx_int_put_block(dst, src, (size_t)n, pe);
  nvshmemx_quiet_block();
  if (threadIdx.x == 0) {
    nvshmemx_signal_op(sig, (uint64_t)n, NVSHMEM_SIGNAL_SET, pe);
    facts[0] = nvshmem_my_pe();
    facts[1] = nvshmem_n_pes();
  }
}
