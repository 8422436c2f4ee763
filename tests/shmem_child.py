"""Child of tests/test_mpi_shmem_bootstrap.py: a program that runs under OpenSHMEM (the stand-in of tests/data/fake_shmem.c,
initialised by the program) brings this library up beside it with NVSHMEMX_INIT_WITH_SHMEM."""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import nvshmem.bindings as b  # noqa: E402

shmem = C.CDLL(os.environ["FAKE_SHMEM_LIB"], mode=C.RTLD_GLOBAL)
shmem.shmem_init()
attr = b.InitAttr()
b.hostlib_init_attr(b.Flags.INIT_WITH_SHMEM, attr.ptr)
assert (b.my_pe(), b.n_pes()) == (shmem.shmem_my_pe(), shmem.shmem_n_pes()) == (int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]))
p = b.calloc(2, 8)
b.barrier_all()
b.free(p)
b.hostlib_finalize()
assert shmem.shmem_n_pes() == int(os.environ["WORLD_SIZE"]), "the bootstrap must not finalise an OpenSHMEM that the program initialised"
shmem.shmem_finalize()
print(f"PE {os.environ['RANK']}: init beside the program's OpenSHMEM ok", flush=True)
