"""Single-node process launcher for programs that call plain ``nvshmem_init()``.

  python -m nvshmem_b200.launch -n 4 [--timeout 300] -- ./examples/bin/ring-reduce

Starts ``n`` copies of the program with ``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK`` and
``NVSHMEM_BOOTSTRAP_UID_SESSION_ID=127.0.0.1:<free port>`` set, which is what the host library's
default bootstrap reads (rank 0 listens on that address, the others connect to it).  The library
directory is put on ``LD_LIBRARY_PATH``.  The role of the reference's ``nvshmrun`` / Hydra launcher
(reference: scripts/install_hydra.sh and the ``nvshmrun -n N`` lines in its examples' comments).

Exit code: 0 when every rank exits 0, else the first non-zero status (124 on timeout).  On failure or
timeout exactly the children started here are terminated.
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
import time
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(n: int, cmd: list[str], timeout: float = 300.0, env_extra: dict | None = None, capture: bool = False) -> tuple[int, list[str]]:
    """Runs `cmd` as n ranks.  Returns (status, per-rank output if capture else [])."""
    session = f"127.0.0.1:{free_port()}"
    procs = []
    for rank in range(n):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "WORLD_SIZE": str(n), "LOCAL_RANK": str(rank), "NVSHMEM_BOOTSTRAP_UID_SESSION_ID": session,
                    "LD_LIBRARY_PATH": f"{LIB_DIR}:" + env.get("LD_LIBRARY_PATH", "")})
        if env_extra:
            env.update(env_extra)
        out = subprocess.PIPE if capture else None
        procs.append(subprocess.Popen(cmd, env=env, stdout=out, stderr=subprocess.STDOUT if capture else None, text=True))
    deadline = time.time() + timeout
    status = 0
    while time.time() < deadline:
        codes = [p.poll() for p in procs]
        if any(c not in (None, 0) for c in codes):
            status = next(c for c in codes if c not in (None, 0))
            break
        if all(c == 0 for c in codes):
            break
        time.sleep(0.05)
    else:
        status = 124
    outputs = []
    for p in procs:
        if p.poll() is None and status != 0:
            p.terminate()  # exactly the child started above
        try:
            o, _ = p.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outputs.append(o or "")
        if status == 0 and p.returncode != 0:
            status = p.returncode
    return status, outputs if capture else []


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-n", "--np", type=int, default=2, dest="n")
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    args = ap.parse_args()
    cmd = args.cmd[1:] if args.cmd and args.cmd[0] == "--" else args.cmd
    if not cmd:
        ap.error("no program given")
    status, _ = launch(args.n, cmd, args.timeout)
    return status


if __name__ == "__main__":
    sys.exit(main())
