"""Runs lists of perftest drivers over PE counts, with time-outs, and collects results and failures.

  python -m perftest.runner --list p2p --npes 2                 # one list, one PE count
  python -m perftest.runner --list all --npes 1,2,4,8 --out results/

A list names driver modules of this package with their arguments.  Every (test, PE count) pair runs
as ``python -m torch.distributed.run --nproc-per-node N -m perftest.<driver> <args>`` (plain
``python -m`` for one PE) with rendezvous on 127.0.0.1, its JSON lines go to
``<out>/<list>_<driver>_n<N>.jsonl``, its full output to a ``.log`` beside it, and a summary
(``summary.json``) records status, duration and row count of each.  Only the started child is ever
terminated on a time-out.  (reference: perftest/perftestRunner.py and perftestCommon.py — test
lists, PE counts, time-outs, failure collection; the launcher there is mpirun / srun.)
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import time
from pathlib import Path

LISTS = {
    # (driver module, arguments, PE counts it supports: None = any)
    "p2p": [("rma", ["--max-bytes", "256M"], (2,)), ("host", [], (2,))],
    "coll": [("coll", ["--max-bytes", "128M", "--algos", "best"], None), ("tile", [], None)],
    "coll-all-algos": [("coll", ["--max-bytes", "32M", "--algos", "all", "--cold"], None)],
    "fused": [("fused", [], None), ("moe", [], None)],
    "kernels": [("kernel_case", ["--kernel", k], (1,)) for k in ("gemm", "gemm_bench", "moe_dispatch", "moe_dispatch_fp8", "moe_combine", "allreduce")],
}
LISTS["all"] = LISTS["p2p"] + LISTS["coll"] + LISTS["fused"] + LISTS["kernels"]


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def command(driver: str, args: list[str], npes: int, python: str = sys.executable) -> list[str]:
    if npes == 1:
        return [python, "-m", f"perftest.{driver}", *args]
    return [python, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={npes}", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
            "-m", f"perftest.{driver}", *args]


def run_one(cmd: list[str], timeout: float, env: dict | None = None) -> tuple[int, str, float]:
    """Runs one command; returns (status, combined output, seconds).  Status 124 = timed out."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, start_new_session=True)
    try:
        out, _ = proc.communicate(timeout=timeout)
        status = proc.returncode
    except subprocess.TimeoutExpired:
        try:
            os.killpg(proc.pid, 15)  # the group of the child started above (torchrun and its ranks)
        except ProcessLookupError:
            pass
        try:
            out, _ = proc.communicate(timeout=15)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, 9)
            out, _ = proc.communicate()
        status = 124
    return status, out or "", time.time() - t0


def run_list(name: str, pe_counts: list[int], out_dir: Path, timeout: float, runner=run_one, python: str = sys.executable) -> list[dict]:
    out_dir.mkdir(parents=True, exist_ok=True)
    summary = []
    for driver, args, allowed in LISTS[name]:
        for n in pe_counts:
            if allowed is not None and n not in allowed:
                continue
            cmd = command(driver, list(args), n, python)
            status, out, secs = runner(cmd, timeout)
            tag = f"{name}_{driver}_{'_'.join(a.strip('-') for a in args if not a.startswith('--'))}_n{n}".replace("__", "_")
            rows = [l for l in out.splitlines() if l.startswith("{")]
            (out_dir / f"{tag}.jsonl").write_text("\n".join(rows) + ("\n" if rows else ""))
            (out_dir / f"{tag}.log").write_text(out)
            entry = {"list": name, "driver": driver, "args": args, "npes": n, "status": status, "seconds": round(secs, 1), "rows": len(rows), "command": " ".join(cmd)}
            summary.append(entry)
            print(f"[{'ok' if status == 0 else 'FAILED ' + str(status)}] {driver} {' '.join(args)} on {n} PE(s): {len(rows)} rows in {secs:.1f} s", flush=True)
    return summary


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--list", default="p2p", choices=sorted(LISTS))
    ap.add_argument("--npes", default="2", help="comma-separated PE counts")
    ap.add_argument("--out", default="perf_out/perftest")
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds per test")
    args = ap.parse_args()
    counts = [int(x) for x in args.npes.split(",") if x]
    out_dir = Path(args.out)
    summary = run_list(args.list, counts, out_dir, args.timeout)
    (out_dir / "summary.json").write_text(json.dumps(summary, indent=1))
    failed = [s for s in summary if s["status"] != 0]
    print(f"{len(summary) - len(failed)} of {len(summary)} runs succeeded" + ("" if not failed else "; failed: " + ", ".join(f"{s['driver']}@{s['npes']}" for s in failed)))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
