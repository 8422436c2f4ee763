"""Child of tests/test_examples.py::test_bootstrap_plugin_collectives: drives the plugin's allgather / alltoall /
barrier directly with odd and large sizes (no heap, no GPU)."""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nvshmem_b200.bindings import host as H  # noqa: E402

lib = H.load()
lib.bshmem_test_boot_init_plugin.restype = C.c_void_p
st = C.c_int(-1)
h = lib.bshmem_test_boot_init_plugin(C.byref(st))
assert h and st.value == 0, st.value
h = C.c_void_p(h)
rank, world = lib.bshmem_test_boot_rank(h), lib.bshmem_test_boot_size(h)
assert rank == int(os.environ["RANK"]) and world == int(os.environ["WORLD_SIZE"])
for nbytes in (1, 33, 4096, 300000):
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
lib.bshmem_test_boot_finalize(h)
if rank == 0:
    print("plugin collectives ok", flush=True)
