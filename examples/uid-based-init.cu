// Initialisation from a unique id that the application distributes itself.  Here rank 0 writes the id
// to a file named by UID_FILE and the others read it; any out-of-band channel (MPI_Bcast, a key-value
// store, torch.distributed) does the same job.
//   UID_FILE=/tmp/uid.bin python -m nvshmem_b200.launch -n 2 -- examples/bin/uid-based-init
// (counterpart of the reference's examples/uid-based-init.cu, which broadcasts the id with MPI)
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

#include "nvshmem.h"
#include "nvshmemx.h"

int main() {
  const char* rank_s = getenv("RANK");
  const char* size_s = getenv("WORLD_SIZE");
  const char* path = getenv("UID_FILE");
  if (!rank_s || !size_s || !path) {
    fprintf(stderr, "set RANK, WORLD_SIZE and UID_FILE\n");
    return 2;
  }
  const int rank = atoi(rank_s), nranks = atoi(size_s);
  cudaSetDevice(rank);  // one GPU per rank on this node
  nvshmemx_uniqueid_t id = NVSHMEMX_UNIQUEID_INITIALIZER;
  char tmp[512];
  snprintf(tmp, sizeof(tmp), "%s.tmp", path);
  if (rank == 0) {
    nvshmemx_get_uniqueid(&id);
    FILE* f = fopen(tmp, "wb");
    fwrite(&id, sizeof(id), 1, f);
    fclose(f);
    rename(tmp, path);  // readers never see a partial file
  } else {
    FILE* f = nullptr;
    for (int tries = 0; tries < 3000 && !(f = fopen(path, "rb")); ++tries) usleep(10000);
    if (!f || fread(&id, sizeof(id), 1, f) != 1) {
      fprintf(stderr, "rank %d: no unique id at %s\n", rank, path);
      return 3;
    }
    fclose(f);
  }
  nvshmemx_init_attr_t attr = NVSHMEMX_INIT_ATTR_INITIALIZER;
  nvshmemx_set_attr_uniqueid_args(rank, nranks, &id, &attr);
  int st = nvshmemx_init_attr(NVSHMEMX_INIT_WITH_UNIQUEID, &attr);
  if (st != 0) {
    fprintf(stderr, "rank %d: init failed with %d\n", rank, st);
    return 4;
  }
  printf("rank %d is PE %d of %d\n", rank, nvshmem_my_pe(), nvshmem_n_pes());
  nvshmem_barrier_all();
  if (rank == 0) unlink(path);
  nvshmem_finalize();
  return 0;
}
