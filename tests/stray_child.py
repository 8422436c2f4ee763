"""Child of tests/test_examples.py::test_stray_connections_do_not_disturb_the_bootstrap: before joining, rank 1
pokes the unique-id root's port twice as a stranger (garbage instead of the job's magic number; a connection that
closes at once).  The root must drop both and the job must still come up."""
import ctypes as C
import os
import socket
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nvshmem_b200.bindings import host as H  # noqa: E402

rank = int(os.environ["RANK"])
host, port = os.environ["NVSHMEM_BOOTSTRAP_UID_SESSION_ID"].rsplit(":", 1)
lib = H.load()
if rank == 1:
    deadline = time.time() + 30
    poked = 0
    while poked < 2 and time.time() < deadline:
        try:
            with socket.create_connection((host, int(port)), timeout=2) as s:
                if poked == 0:
                    s.sendall(os.urandom(8) + b"not a registration" * 8)
                poked += 1
        except OSError:
            time.sleep(0.05)  # the root (started by rank 0) is not listening yet
    assert poked == 2, "could not reach the root's port"
lib.nvshmem_init()
assert lib.nvshmemx_init_status() >= 2 and lib.nvshmem_n_pes() == int(os.environ["WORLD_SIZE"])
lib.nvshmem_barrier_all()
lib.nvshmem_finalize()
if rank == 0:
    print("bootstrap survived the strays", flush=True)
