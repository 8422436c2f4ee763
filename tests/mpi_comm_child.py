"""Child of tests/test_mpi_shmem_bootstrap.py: a program that has initialised MPI itself hands its communicator to the
library (NVSHMEMX_INIT_WITH_MPI_COMM through the pointer-level bindings), works on the host-memory heap, and
finalises MPI itself afterwards.  The MPI library is the stand-in built from tests/data/fake_mpi.c."""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import nvshmem.bindings as b  # noqa: E402

mpi = C.CDLL(os.environ["FAKE_MPI_LIB"], mode=C.RTLD_GLOBAL)  # in the process before the bootstrap looks for it
assert mpi.MPI_Init(None, None) == 0
if os.environ["FAKE_MPI_ABI"] == "ompi":
    comm = C.c_void_p(C.addressof(C.c_char.in_dll(mpi, "ompi_mpi_comm_world")))
else:
    comm = C.c_int(0x44000000)
if os.environ.get("USE_CORE_LAYER") == "1":  # the same through nvshmem.core.init(mpi_comm=...)
    import nvshmem.core as nv
    nv.init(mpi_comm=comm, initializer_method="mpi")
    assert nv.is_initialized()
else:
    attr = b.InitAttr()
    b.set_attr_mpi_comm_args(C.addressof(comm), attr.ptr)
    assert attr.mpi_comm == C.addressof(comm)
    b.hostlib_init_attr(b.Flags.INIT_WITH_MPI_COMM, attr.ptr)
rank, size = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
assert (b.my_pe(), b.n_pes()) == (rank, size)
p = b.calloc(4, 8)
b.barrier_all()
b.putmem_on_stream(p + 8 * 0, p + 8 * 1, 8, (rank + 1) % size, 0)   # zeros over zeros: exercises the path only
b.barrier_all()
b.free(p)
if os.environ.get("USE_CORE_LAYER") == "1":
    nv.finalize()
else:
    b.hostlib_finalize()
flag = C.c_int(-1)
mpi.MPI_Finalized(C.byref(flag))
assert flag.value == 0, "the bootstrap must not finalise an MPI that the program initialised"
mpi.MPI_Finalize()
print(f"rank {rank}: init with the program's communicator ok", flush=True)
