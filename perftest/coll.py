"""Collectives: on-stream (one launch per call, also replayed from a CUDA graph), device-initiated
(block scope, many calls per launch) and barrier / sync latency, for every algorithm, against NCCL on
the same GPUs.  Reports latency and bus bandwidth.

  torchrun --nproc-per-node 8 -m perftest.coll [--max-bytes 1G] [--dtypes bf16,fp32]
(reference counterparts: perftest/host/coll/*_on_stream, perftest/device/coll/*_latency)
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch
import torch.distributed as dist

from .common import Env, busbw_factor, sizes_pow2, stream_ptr, ok
from .rma import parse_size


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--graph", action="store_true", help="also time the collectives replayed from a CUDA graph")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--c-loop", action="store_true", help="also issue the automatic choice of each on-stream call from a C loop (eager, no interpreter between launches)")
    ap.add_argument("--cold", action="store_true", help="also time single calls with the L2 flushed before each (8 MB and up)")
    ap.add_argument("--algos", default="all", help="'all' or 'best': only the automatic choice of each collective")
    args = ap.parse_args()
    env = Env()
    nv = env.nv
    n = env.world
    nvls = nv.heap_info()["mc_base"] != 0
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    dts = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}
    src = nv.tensor((hi,), torch.uint8)
    dst = nv.tensor((hi,), torch.uint8)
    src.random_(0, 100)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=env.dev)
    flush = lambda: flush_buf.zero_()

    def run(name, algo, dtype_name, size, fn, factor_name, per_pe_bytes):
        # `us`: calls issued back to back, as the reference's perftest loops do.  The library's own calls are
        # replayed from a CUDA graph so that no Python time sits between launches; NCCL goes through torch eagerly.
        # `cold_us` (8 MB and up): one call at a time with the L2 flushed before it; includes the ranks' skew.
        iters = 20 if size <= (16 << 20) else 8
        if algo == "nccl":
            ms, how = env.time_ms(lambda: fn(None), iters=iters, warmup=3), "eager"
        else:
            ms, how = env.time_graph_ms(fn, iters=iters), "graph"
        extra = {}
        if size >= (8 << 20) and args.cold:
            extra["cold_us"] = round(env.time_ms(lambda: fn(None), iters=5, warmup=1, flush=flush) * 1e3, 2)
        bw = per_pe_bytes / (ms * 1e-3) / 1e9
        env.record(test=name, algo=algo, dtype=dtype_name, bytes_per_pe=size, us=round(ms * 1e3, 2), algbw_GBps=round(bw, 2),
                   busbw_GBps=round(bw * busbw_factor(factor_name, n), 2), npes=n, nvls=nvls, issue=how, **extra)

    def pick(lst):
        return ["auto"] if args.algos == "best" else lst + ["auto"]

    for dname in args.dtypes.split(","):
        dt = dts[dname]
        es = torch.empty((), dtype=dt).element_size()
        for size in sizes_pow2(lo, hi):
            cnt = size // es
            s, d = src[:size].view(dt), dst[:size].view(dt)
            # allreduce: `size` bytes per PE
            for algo in pick(["oneshot", "twoshot"] + (["nvls_oneshot", "nvls_twoshot"] if nvls else [])):
                if algo in ("oneshot", "nvls_oneshot") and size > (4 << 20):
                    continue
                run("allreduce_on_stream", algo, dname, size, lambda st: nv.reduce(0, d, s, "sum", algo=algo, stream=st), "allreduce", size)
            if not args.no_nccl and n > 1:
                t = torch.empty(cnt, dtype=dt, device=env.dev)
                run("allreduce_nccl", "nccl", dname, size, lambda st: dist.all_reduce(t), "allreduce", size)
            # reducescatter / fcollect / alltoall: `size` bytes is the full buffer, size/n per block
            if cnt % n == 0 and cnt >= n:
                blk = cnt // n
                for algo in pick(["pull"] + (["nvls"] if nvls else [])):
                    run("reducescatter_on_stream", algo, dname, size, lambda st: nv.reducescatter(0, d[:blk], s, "sum", algo=algo, stream=st), "reducescatter", size)
                for algo in pick(["push"] + (["ll"] if size // n <= 2048 else []) + (["nvls"] if nvls else [])):
                    run("fcollect_on_stream", algo, dname, size, lambda st: nv.fcollect(0, d, s[:blk], algo=algo, stream=st), "fcollect", size)
                run("alltoall_on_stream", "push", dname, size, lambda st: nv.alltoall(0, d, s, stream=st), "alltoall", size)
                if not args.no_nccl and n > 1:
                    full, part = torch.empty(cnt, dtype=dt, device=env.dev), torch.empty(blk, dtype=dt, device=env.dev)
                    run("reducescatter_nccl", "nccl", dname, size, lambda st: dist.reduce_scatter_tensor(part, full), "reducescatter", size)
                    run("allgather_nccl", "nccl", dname, size, lambda st: dist.all_gather_into_tensor(full, part), "fcollect", size)
                    full2 = torch.empty(cnt, dtype=dt, device=env.dev)
                    run("alltoall_nccl", "nccl", dname, size, lambda st: dist.all_to_all_single(full2, full), "alltoall", size)
            for algo in pick(["push", "pull"] + (["nvls"] if nvls else [])):
                run("broadcast_on_stream", algo, dname, size, lambda st: nv.broadcast(0, d, s, root=0, algo=algo, stream=st), "broadcast", size)
        break_after_first = False
    # barrier / sync latency: on-stream and device-initiated
    lib = env.devlib()
    if args.c_loop:
        # The same calls issued eagerly from C, as the reference's host perftests issue theirs.
        lib.perf_onstream_loop.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
        kinds = ((0, "allreduce_on_stream", "allreduce"), (1, "reducescatter_on_stream", "reducescatter"), (2, "fcollect_on_stream", "fcollect"),
                 (3, "alltoall_on_stream", "alltoall"), (4, "broadcast_on_stream", "broadcast"))
        for size in sizes_pow2(lo, hi):
            if size % (4 * n):
                continue
            iters = 20 if size <= (16 << 20) else 8
            for kind, name, fac in kinds:
                ms = env.time_ms(lambda: ok(lib.perf_onstream_loop(kind, C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), size, 0, iters, stream_ptr())), iters=3, warmup=1)
                us = ms * 1e3 / iters
                env.record(test=name, algo="auto", dtype="fp32", bytes_per_pe=size, us=round(us, 2), busbw_GBps=round(size / (us * 1e-6) / 1e9 * busbw_factor(fac, n), 2),
                           npes=n, nvls=nvls, issue="c-loop")
        for kind, name in ((5, "barrier_all_on_stream"), (6, "sync_all_on_stream")):
            ms = env.time_ms(lambda: ok(lib.perf_onstream_loop(kind, None, None, 0, 0, 100, stream_ptr())), iters=3, warmup=1)
            env.record(test=name, us=round(ms * 1e3 / 100, 2), npes=n, issue="c-loop")
    ms = env.time_graph_ms(lambda st: nv.barrier_all(stream=st), iters=50)
    env.record(test="barrier_all_on_stream", us=round(ms * 1e3, 2), npes=n, issue="graph")
    ms = env.time_graph_ms(lambda st: nv.sync_all(stream=st), iters=50)
    env.record(test="sync_all_on_stream", us=round(ms * 1e3, 2), npes=n, issue="graph")
    ms = env.time_ms(lambda: nv.barrier_all(), iters=50, warmup=5)
    env.record(test="barrier_all_on_stream", us=round(ms * 1e3, 2), npes=n, issue="eager")
    for scope, sname in ((0, "thread"), (1, "warp"), (2, "block")):
        for sync_only in (0, 1):
            iters = 200
            ms = env.time_ms(lambda: ok(lib.perf_barrier_latency(iters, scope, sync_only, 256, stream_ptr())), iters=3, warmup=1)
            env.record(test="sync_device" if sync_only else "barrier_device", scope=sname, us=round(ms * 1e3 / iters, 3), npes=n)
    # device-initiated collectives (block scope), small and medium sizes
    fsrc, fdst = src.view(torch.float32), dst.view(torch.float32)
    for kind, kname, fac in ((0, "allreduce_device_fp32", "allreduce"), (2, "reducescatter_device_fp32", "reducescatter"), (3, "fcollect_device_int", "fcollect"),
                             (4, "alltoall_device_int", "alltoall"), (5, "broadcast_device_int", "broadcast"), (6, "allreduce_device_bf16", "allreduce")):
        for cnt in (16, 256, 4096, 65536, 1 << 20):
            es = 2 if kind == 6 else 4
            nel = cnt // n if kind in (2, 3, 4) else cnt
            if nel < 1 or cnt * es > hi:
                continue
            iters = 50 if cnt <= 65536 else 10
            ms = env.time_ms(lambda: ok(lib.perf_coll_latency(kind, C.c_void_p(fdst.data_ptr()), C.c_void_p(fsrc.data_ptr()), C.c_size_t(nel), iters, 1024, stream_ptr())), iters=3, warmup=1)
            us = ms * 1e3 / iters
            env.record(test=kname, bytes=cnt * es, us=round(us, 2), busbw_GBps=round(cnt * es / (us * 1e-6) / 1e9 * busbw_factor(fac, n), 2), npes=n)
    # CUDA-graph replay of an on-stream allreduce + barrier
    if args.graph:
        s32, d32 = src[:1 << 20].view(torch.float32), dst[:1 << 20].view(torch.float32)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            nv.reduce(0, d32, s32, "sum", stream=stream)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(10):
                    nv.reduce(0, d32, s32, "sum", stream=stream)
        ms = env.time_ms(lambda: g.replay(), iters=10, warmup=2)
        env.record(test="allreduce_on_stream_graph", dtype="fp32", bytes_per_pe=1 << 20, us=round(ms * 1e3 / 10, 2), npes=n)
    env.barrier()
    nv.free_tensor(src)
    nv.free_tensor(dst)
    env.finish()


if __name__ == "__main__":
    main()
