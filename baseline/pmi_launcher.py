"""A minimal PMI-1 ("simple PMI") and PMI-2 process manager, enough to start the UNMODIFIED reference perftest
binaries of ``baseline/_ref`` on the GPUs of one node without MPI, Hydra or Slurm.  A client that opens with
``cmd=init pmi_version=2`` is served the PMI-2 wire protocol from then on (6-digit length + ``cmd=..;key=value;``
messages: fullinit, job-getid, kvs-put, kvs-get, kvs-fence, finalize, abort).

The reference programs call ``nvshmem_init()``, whose default bootstrap is PMI: each process finds a
socket in ``PMI_FD`` and speaks a line protocol (init, get_maxes, get_my_kvsname, put, get, barrier_in,
finalize).  This launcher creates one socket pair per rank, starts the ranks with ``PMI_FD``,
``PMI_RANK`` and ``PMI_SIZE`` set, and serves those commands from a single select loop.

  python -m baseline.pmi_launcher -n 2 [--timeout 300] -- baseline/_ref/bin/perftest/device/pt-to-pt/shmem_put_bw -b 8 -e 64M

Exit code: 0 when every rank exits 0.  On timeout exactly the started children are killed.
"""
from __future__ import annotations

import argparse
import os
import select
import socket
import subprocess
import sys
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def parse(line: str) -> dict:
    out = {}
    for tok in line.strip().split(" "):
        if "=" in tok:
            k, v = tok.split("=", 1)
            out[k] = v
    return out


def launch(n: int, cmd: list[str], timeout: float = 300.0, env_extra: dict | None = None, quiet: bool = False) -> tuple[int, str]:
    """Runs `cmd` as n PMI ranks.  Returns (exit status, combined output of rank 0)."""
    kvs: dict[str, str] = {}
    socks, procs, bufs = [], [], []
    in_barrier: set[int] = set()
    v2: set[int] = set()        # connections that negotiated PMI-2
    in_fence: set[int] = set()
    for rank in range(n):
        parent, child = socket.socketpair()
        env = dict(os.environ)
        env.update({"PMI_FD": str(child.fileno()), "PMI_RANK": str(rank), "PMI_SIZE": str(n), "NVSHMEM_BOOTSTRAP": "PMI",
                    "LD_LIBRARY_PATH": f"{REF / 'lib'}:" + env.get("LD_LIBRARY_PATH", "")})
        if env_extra:
            env.update(env_extra)
        out = subprocess.PIPE if rank == 0 else subprocess.DEVNULL
        procs.append(subprocess.Popen(cmd, env=env, pass_fds=(child.fileno(),), stdout=out, stderr=subprocess.STDOUT if rank == 0 else subprocess.DEVNULL, text=True))
        child.close()
        parent.setblocking(False)
        socks.append(parent)
        bufs.append(b"")
    deadline = time.time() + timeout
    live = set(range(n))

    def reply(i: int, text: str) -> None:
        try:
            socks[i].sendall(text.encode())
        except OSError:
            pass

    def handle(i: int, line: str) -> None:
        kv = parse(line)
        c = kv.get("cmd", "")
        if c == "init":
            if kv.get("pmi_version") == "2":
                v2.add(i)
                reply(i, "cmd=response_to_init pmi_version=2 pmi_subversion=0 rc=0\n")
            else:
                reply(i, "cmd=response_to_init pmi_version=1 pmi_subversion=1 rc=0\n")
        elif c == "get_maxes":
            reply(i, "cmd=maxes kvsname_max=256 keylen_max=256 vallen_max=1024\n")
        elif c == "get_my_kvsname":
            reply(i, "cmd=my_kvsname kvsname=kvs_ref_0\n")
        elif c == "get_appnum":
            reply(i, "cmd=appnum appnum=0\n")
        elif c == "get_universe_size":
            reply(i, f"cmd=universe_size size={n}\n")
        elif c == "put":
            kvs[kv.get("key", "")] = kv.get("value", "")
            reply(i, "cmd=put_result rc=0 msg=success\n")
        elif c == "get":
            key = kv.get("key", "")
            if key in kvs:
                reply(i, f"cmd=get_result rc=0 msg=success value={kvs[key]}\n")
            else:
                reply(i, f"cmd=get_result rc=-1 msg=key_{key}_not_found value=unknown\n")
        elif c == "barrier_in":
            in_barrier.add(i)
            if len(in_barrier) == n:
                for j in in_barrier:
                    reply(j, "cmd=barrier_out\n")
                in_barrier.clear()
        elif c == "finalize":
            reply(i, "cmd=finalize_ack\n")
        elif c == "abort":
            for p in procs:
                if p.poll() is None:
                    p.kill()

    def reply2(i: int, body: str) -> None:
        reply(i, f"{len(body):6d}{body}")

    def handle2(i: int, body: str) -> None:
        kv = dict(tok.split("=", 1) for tok in body.split(";") if "=" in tok)
        c = kv.get("cmd", "")
        if c == "fullinit":
            reply2(i, f"cmd=fullinit-response;pmi-version=2;pmi-subversion=0;rank={kv.get('pmirank', i)};size={n};appnum=0;debugged=FALSE;pmiverbose=FALSE;rc=0;")
        elif c == "job-getid":
            reply2(i, "cmd=job-getid-response;jobid=kvs_ref_0;rc=0;")
        elif c == "kvs-put":
            kvs[kv.get("key", "")] = kv.get("value", "")
            reply2(i, "cmd=kvs-put-response;rc=0;")
        elif c == "kvs-get":
            key = kv.get("key", "")
            if key in kvs:
                reply2(i, f"cmd=kvs-get-response;found=TRUE;value={kvs[key]};rc=0;")
            else:
                reply2(i, "cmd=kvs-get-response;found=FALSE;rc=0;")
        elif c == "kvs-fence":
            in_fence.add(i)
            if len(in_fence) == n:
                for j in in_fence:
                    reply2(j, "cmd=kvs-fence-response;rc=0;")
                in_fence.clear()
        elif c == "finalize":
            reply2(i, "cmd=finalize-response;rc=0;")
        elif c == "abort":
            for p in procs:
                if p.poll() is None:
                    p.kill()

    while live and time.time() < deadline:
        ready, _, _ = select.select([socks[i] for i in live], [], [], 0.2)
        for s in ready:
            i = socks.index(s)
            try:
                data = s.recv(65536)
            except BlockingIOError:
                continue
            except OSError:
                data = b""
            if not data:
                live.discard(i)
                continue
            bufs[i] += data
            while True:
                if i in v2 and bufs[i][:4] == b"cmd=":
                    v2.discard(i)  # a client that finalized and initialises again opens with a PMI-1 style line
                if i in v2:
                    if len(bufs[i]) < 6:
                        break
                    try:
                        ln = int(bufs[i][:6])
                    except ValueError:
                        bufs[i] = b""
                        break
                    if len(bufs[i]) < 6 + ln:
                        break
                    body, bufs[i] = bufs[i][6:6 + ln], bufs[i][6 + ln:]
                    handle2(i, body.decode(errors="replace"))
                else:
                    if b"\n" not in bufs[i]:
                        break
                    line, bufs[i] = bufs[i].split(b"\n", 1)
                    handle(i, line.decode(errors="replace"))
        for i in list(live):
            if procs[i].poll() is not None and not select.select([socks[i]], [], [], 0)[0]:
                live.discard(i)
        if any(p.poll() not in (None, 0) for p in procs):
            break
    status = 0
    out0 = ""
    for i, p in enumerate(procs):
        try:
            o, _ = p.communicate(timeout=max(1.0, min(20.0, deadline - time.time())))
        except subprocess.TimeoutExpired:
            p.kill()  # exactly the child started above
            o, _ = p.communicate()
            status = status or 124
        if i == 0:
            out0 = o or ""
        if p.returncode != 0:
            status = status or (p.returncode if p.returncode else 1)
    for s in socks:
        s.close()
    if not quiet:
        sys.stdout.write(out0)
    return status, out0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("-n", type=int, default=2)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    args = ap.parse_args()
    cmd = args.cmd[1:] if args.cmd and args.cmd[0] == "--" else args.cmd
    if not cmd:
        ap.error("no command")
    status, _ = launch(args.n, cmd, args.timeout)
    return status


if __name__ == "__main__":
    sys.exit(main())
