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
        if not gpu:
            e["CUDA_VISIBLE_DEVICES"] = ""
            e.setdefault("NVSHMEM_SYMMETRIC_SIZE", "16M")
        if env:
            e.update(env)
        procs.append(subprocess.Popen([sys.executable, "-m", "tests.workers", func] + (args or []), cwd=ROOT, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    deadline = time.time() + timeout
    outs, codes = [], []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=max(1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            p.kill()  # exactly the child we started
            out, _ = p.communicate()
            out += "\n[killed: timeout]"
        outs.append(out)
        codes.append(p.returncode)
    if not expect_fail:
        assert all(c == 0 for c in codes), "worker failed:\n" + "\n".join(f"--- rank {i} rc={c}\n{o[-3000:]}" for i, (c, o) in enumerate(zip(codes, outs)))
    return codes, outs
