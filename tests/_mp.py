"""Runs a worker function from tests/workers.py in N child processes (one per rank / GPU)."""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(func: str, nprocs: int, gpu: bool = False, env: dict | None = None, timeout: int = 300, expect_fail: bool = False, args: list[str] | None = None):
    port = free_port()
    procs = []
    for rank in range(nprocs):
        e = dict(os.environ)
        e.update({"RANK": str(rank), "WORLD_SIZE": str(nprocs), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                  "BSHMEM_TEST_GPU": "1" if gpu else "0", "PYTHONPATH": ROOT + os.pathsep + e.get("PYTHONPATH", "")})
        e.setdefault("NVSHMEM_WAIT_TIMEOUT_MS", "5000")  # a lost peer costs seconds, not minutes
        if not gpu:
            e["CUDA_VISIBLE_DEVICES"] = ""
            e.setdefault("NVSHMEM_SYMMETRIC_SIZE", "16M")
        if env:
            e.update(env)
        procs.append(subprocess.Popen([sys.executable, "-m", "tests.workers", func] + (args or []), cwd=ROOT, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    deadline = time.time() + timeout
    # Fail fast: once a rank has exited with an error the others can only time out, so give them a
    # short grace period and stop exactly the children started here.
    # A rank whose heap is bound to an NVLink multicast object is never killed outright: it gets SIGTERM, which the
    # worker turns into "detach from the multicast objects, then exit", and a grace period longer than the bound
    # of the device-side waits, so that it leaves by itself.  SIGKILL right away is for runs with NVLS off only.
    nvls_may_be_on = gpu and (env or {}).get("NVSHMEM_DISABLE_NVLS") != "1"
    grace = 45 if nvls_may_be_on else 15
    first_failure = None
    terminated_at = None
    while True:
        codes = [p.poll() for p in procs]
        if all(c is not None for c in codes):
            break
        now = time.time()
        if first_failure is None and any(c not in (None, 0) for c in codes):
            first_failure = now
        if terminated_at is None and (now > deadline or (first_failure is not None and now - first_failure > 15)):
            terminated_at = now
            for p in procs:
                if p.poll() is None:
                    p.terminate() if nvls_may_be_on else p.kill()
        if terminated_at is not None and now - terminated_at > grace:
            for p in procs:
                if p.poll() is None:
                    p.kill()
            break
        time.sleep(0.2)
    outs, codes = [], []
    for p in procs:
        out, _ = p.communicate()
        outs.append(out)
        codes.append(p.returncode)
    if not expect_fail:
        order = sorted(range(nprocs), key=lambda i: (codes[i] in (0, -9, -15), i))  # the rank that failed by itself first
        assert all(c == 0 for c in codes), "worker failed:\n" + "\n".join(f"--- rank {i} rc={codes[i]}\n{outs[i][-2500:]}" for i in order)
    return codes, outs
