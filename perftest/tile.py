"""Tile collectives from inside a kernel (block scope): all-reduce (one-shot and two-shot) and all-gather latency
over tile sizes, fp32.

  torchrun --nproc-per-node 8 -m perftest.tile [--max-cols 4096]
(reference counterparts: perftest/device/tile/tile_allreduce_latency.cu, tile_allgather_latency.cu)
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from .common import Env, busbw_factor, ok, stream_ptr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--max-cols", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    env = Env()
    nv, n = env.nv, env.world
    lib = env.devlib()
    lib.perf_tile_latency.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    rows, ld = args.rows, args.max_cols
    src = nv.tensor((rows * ld,), torch.float32)
    dst = nv.tensor((rows * ld * max(n, 1),), torch.float32)  # the all-gather's destination holds n tiles
    src.fill_(1.0)
    cols = 32
    while cols <= args.max_cols:
        for kind, name, fac in ((0, "tile_allreduce_oneshot", "allreduce"), (1, "tile_allreduce_twoshot", "allreduce"), (2, "tile_allgather", "fcollect")):
            nv.barrier_all()
            ms = env.time_ms(lambda: ok(lib.perf_tile_latency(kind, C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), rows, cols, ld, args.iters, 1024, stream_ptr())),
                             iters=3, warmup=1)
            us = ms * 1e3 / args.iters
            nbytes = rows * cols * 4 * (n if kind == 2 else 1)
            env.record(test=name, rows=rows, cols=cols, bytes=nbytes, us=round(us, 2), busbw_GBps=round(nbytes / (us * 1e-6) / 1e9 * busbw_factor(fac, n), 2), npes=n)
        cols *= 4
    env.barrier()
    nv.free_tensor(src)
    nv.free_tensor(dst)
    env.finish()


if __name__ == "__main__":
    main()
