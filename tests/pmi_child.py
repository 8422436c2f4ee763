"""Child process of tests/test_pmi_bootstrap.py: started by a PMI process manager, it drives the PMI
bootstrap's collectives directly (no heap, no GPU) and then a full initialisation on the host heap."""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nvshmem_b200.bindings import host as H  # noqa: E402

lib = H.load()
lib.bshmem_test_boot_init_pmi.restype = C.c_void_p
st = C.c_int(-1)
h = lib.bshmem_test_boot_init_pmi(C.byref(st))
assert h and st.value == 0, st.value
h = C.c_void_p(h)
rank, world = lib.bshmem_test_boot_rank(h), lib.bshmem_test_boot_size(h)
assert rank == int(os.environ["PMI_RANK"]) and world == int(os.environ["PMI_SIZE"])
for nbytes in (1, 33, 448, 449, 3000):  # below, at and above one key-value piece
    send = bytes([(rank * 7 + i) % 251 for i in range(nbytes)])
    recv = C.create_string_buffer(nbytes * world)
    assert lib.bshmem_test_boot_allgather(h, send, recv, nbytes) == 0
    for r in range(world):
        assert recv.raw[r * nbytes:(r + 1) * nbytes] == bytes([(r * 7 + i) % 251 for i in range(nbytes)]), (nbytes, r)
    a2a_send = b"".join(bytes([(rank * 16 + p + i) % 256 for i in range(nbytes)]) for p in range(world))
    a2a_recv = C.create_string_buffer(nbytes * world)
    assert lib.bshmem_test_boot_alltoall(h, a2a_send, a2a_recv, nbytes) == 0
    for p in range(world):
        assert a2a_recv.raw[p * nbytes:(p + 1) * nbytes] == bytes([(p * 16 + rank + i) % 256 for i in range(nbytes)]), (nbytes, p)
    assert lib.bshmem_test_boot_barrier(h) == 0
mn, nn = C.c_int(), C.c_int()
lib.bshmem_test_boot_node_info(h, C.byref(mn), C.byref(nn))
assert nn.value == world and mn.value == rank
if rank == 0:
    print(f"pmi collectives ok on {world} ranks", flush=True)
# Leave the raw handle open (the manager's socket is shared) and run the whole library on top of the same manager.
lib.nvshmem_init()
assert lib.nvshmemx_init_status() >= 2 and lib.nvshmem_my_pe() == rank and lib.nvshmem_n_pes() == world
lib.nvshmem_barrier_all()
p = lib.nvshmem_malloc(4096)
assert p
lib.nvshmem_long_p(C.c_void_p(p), rank + 100, (rank + 1) % world)
lib.nvshmem_barrier_all()
assert lib.nvshmem_long_g(C.c_void_p(p), rank) == (rank + world - 1) % world + 100
lib.nvshmem_free(C.c_void_p(p))
lib.nvshmem_finalize()
if rank == 0:
    print("full init over pmi ok", flush=True)
