"""Runs the UNMODIFIED reference perftest binaries (``baseline/_ref/bin/perftest``) through the PMI
launcher and stores their own output under ``--out`` (default ``perf_out/ref_perftest/``).  These are the numbers the
library's own perftest drivers are compared with.

  python -m baseline.reference_perftest --npes 2 --group p2p          # put/get/signal/atomic, 2 PEs
  python -m baseline.reference_perftest --npes 8 --group coll         # on-stream + device collectives
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from pathlib import Path

from .pmi_launcher import REF, launch

# Point-to-point, config (b): put / get at thread, warp and block scope, 8 B - 1 GB.  Messages up to 64 MB run the
# configured 1000 iterations after 100 warm-up iterations; 128 MB - 1 GB run 100 after 10, which keeps every binary
# inside its time limit (a 1 GB message at thread scope takes milliseconds per iteration).
_BW_SMALL = ["-b", "8", "-e", "64M", "-n", "1000", "-w", "100", "-c", "32", "-t", "1024"]
_BW_LARGE = ["-b", "128M", "-e", "1G", "-n", "100", "-w", "10", "-c", "32", "-t", "1024"]
P2P = [(f"device/pt-to-pt/shmem_{d}_bw", rng + ["-s", sc]) for d in ("put", "get") for sc in ("block", "warp", "thread") for rng in (_BW_SMALL, _BW_LARGE)] + [
    ("device/pt-to-pt/shmem_st_bw", _BW_SMALL),
    ("device/pt-to-pt/shmem_p_bw", ["-b", "8", "-e", "64M", "-n", "1000", "-w", "100", "-c", "32", "-t", "1024"]),
    ("device/pt-to-pt/shmem_g_bw", ["-b", "8", "-e", "64M", "-n", "1000", "-w", "100", "-c", "32", "-t", "1024"]),
    ("device/pt-to-pt/shmem_put_latency", ["-b", "8", "-e", "1M", "-n", "1000", "-w", "100"]),
    ("device/pt-to-pt/shmem_get_latency", ["-b", "8", "-e", "1M", "-n", "1000", "-w", "100"]),
    ("device/pt-to-pt/shmem_p_latency", ["-n", "1000", "-w", "100"]),
    ("device/pt-to-pt/shmem_g_latency", ["-n", "1000", "-w", "100"]),
    ("device/pt-to-pt/shmem_put_signal_ping_pong_latency", ["-b", "8", "-e", "1M", "-n", "500", "-w", "20"]),
    ("device/pt-to-pt/shmem_signal_ping_pong_latency", ["-n", "1000", "-w", "100"]),
] + [("device/pt-to-pt/shmem_atomic_bw", ["-a", a, "-b", "8", "-e", "1M", "-n", "500", "-w", "50", "-c", "32", "-t", "256"])
     for a in ("fetch_add", "add", "compare_swap", "swap", "fetch_or", "inc", "fetch_inc", "and", "fetch_and", "or", "xor", "fetch_xor", "set")] + [
    ("device/pt-to-pt/shmem_atomic_latency", ["-a", "fetch_add", "-n", "1000", "-w", "100"]),
    ("host/pt-to-pt/bw", ["-b", "1K", "-e", "1G", "-n", "20", "-w", "2"]),
    ("host/pt-to-pt/latency", ["-b", "8", "-e", "1M", "-n", "100", "-w", "10"]),
]
# Collectives, config (c): on-stream calls 1 KB - 1 GB on bfloat16 and float (the binaries' own eager C loops), and
# the device-initiated tests.
_CS = ["-b", "1K", "-e", "1G", "-n", "20", "-w", "3"]
COLL = [
    ("host/coll/reduction_on_stream", _CS + ["-d", "bfloat16", "-o", "sum"]),
    ("host/coll/reduction_on_stream", _CS + ["-d", "float", "-o", "sum"]),
    ("host/coll/reducescatter_on_stream", _CS + ["-d", "bfloat16", "-o", "sum"]),
    ("host/coll/reducescatter_on_stream", _CS + ["-d", "float", "-o", "sum"]),
    ("host/coll/fcollect_on_stream", _CS),
    ("host/coll/alltoall_on_stream", _CS),
    ("host/coll/broadcast_on_stream", ["-b", "1K", "-e", "64M", "-n", "20", "-w", "3"]),
    ("host/coll/barrier_all_on_stream", ["-n", "100", "-w", "10"]),
    ("host/coll/sync_all_on_stream", ["-n", "100", "-w", "10"]),
    ("device/coll/reduction_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5", "-d", "float", "-o", "sum"]),
    ("device/coll/reduction_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5", "-d", "bfloat16", "-o", "sum"]),
    ("device/coll/reducescatter_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5", "-d", "float", "-o", "sum"]),
    ("device/coll/barrier_latency", ["-n", "200", "-w", "20"]),
    ("device/coll/sync_latency", ["-n", "200", "-w", "20"]),
    ("device/coll/fcollect_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5"]),
    ("device/coll/alltoall_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5"]),
    ("device/coll/bcast_latency", ["-b", "4", "-e", "4M", "-n", "50", "-w", "5"]),
]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--npes", type=int, default=2)
    ap.add_argument("--group", default="p2p", choices=["p2p", "coll"])
    ap.add_argument("--timeout", type=float, default=180.0)
    ap.add_argument("--only", default="")
    ap.add_argument("--out", default="perf_out/ref_perftest")
    args = ap.parse_args()
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    if not (REF / "bin" / "perftest").exists():
        print("no reference build under baseline/_ref")
        return 0
    failures = 0
    for i, (rel, opts) in enumerate(P2P if args.group == "p2p" else COLL):
        if args.only and args.only not in rel:
            continue
        exe = REF / "bin" / "perftest" / rel
        t0 = time.time()
        status, out = launch(args.npes, [str(exe)] + opts, timeout=args.timeout, env_extra={"NVSHMEM_SYMMETRIC_SIZE": "4G"}, quiet=True)
        tag = f"{rel.replace('/', '_')}_{i}_n{args.npes}"
        (out_dir / f"{tag}.txt").write_text(f"# {exe.name} {' '.join(opts)}  (npes={args.npes}, status={status}, {time.time() - t0:.1f}s)\n{out}")
        print(f"{tag}: status {status}, {time.time() - t0:.1f}s, {len(out.splitlines())} lines", flush=True)
        failures += status != 0
    return 0


if __name__ == "__main__":
    sys.exit(main())
