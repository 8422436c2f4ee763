"""Collectives: on-stream calls for every algorithm, device-initiated calls at thread / warp / block scope, barrier
and sync latency, against NCCL on the same GPUs.  Reports latency and bus bandwidth.

With no arguments: allreduce, reducescatter, fcollect, alltoall and broadcast on bfloat16 and float, 1 KB - 1 GB
per PE in powers of two, every algorithm (one-shot, two-shot, NVLS, flag-in-data) plus the automatic choice.
On-stream calls are issued back to back from a C loop, eagerly, exactly as the reference's host perftests issue
theirs (`"issue": "c-loop"`); `--cudagraph` replays them from a CUDA graph instead (the reference's flag of the
same name).  The argument set is the reference's (-b -e -f -n -w -d -o -s --cudagraph).

  torchrun --nproc-per-node 8 -m perftest.coll [-b 1K -e 1G -d bfloat16,float --algos all|best]
(reference counterparts: perftest/host/coll/*_on_stream, perftest/device/coll/*_latency, redmaxloc_latency)
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch
import torch.distributed as dist

from .common import Env, add_reference_args, busbw_factor, ok, parse_size, scopes_of, sizes_geometric, stream_ptr

DTYPES = {"bfloat16": (torch.bfloat16, 9), "bf16": (torch.bfloat16, 9), "float": (torch.float32, 10), "fp32": (torch.float32, 10), "half": (torch.float16, 8),
          "fp16": (torch.float16, 8), "int": (torch.int32, 4), "int32": (torch.int32, 4), "long": (torch.int64, 6), "double": (torch.float64, 11)}
RED = {"oneshot": 1, "twoshot": 2, "nvls_oneshot": 3, "nvls_twoshot": 4, "ll": 5, "ll128": 6, "auto": 0}
RS = {"pull": 1, "nvls": 2, "auto": 0}
FC = {"push": 1, "ll": 2, "nvls": 3, "ll128": 4, "auto": 0}
BC = {"push": 1, "ll": 2, "nvls": 3, "pull": 4, "auto": 0}


def main():
    ap = argparse.ArgumentParser()
    add_reference_args(ap, min_size="1K", max_size="1G", iters=0, warmup=3)
    ap.add_argument("--dtypes", default=None, help="alias of -d")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--cold", action="store_true", help="also time single calls with the L2 flushed before each (8 MB and up)")
    ap.add_argument("--algos", default="all", help="'all' or 'best': only the automatic choice of each collective")
    ap.add_argument("--tests", default="all", help="comma list of: on_stream, barrier, device")
    args = ap.parse_args()
    env = Env()
    nv = env.nv
    n = env.world
    nvls = nv.heap_info()["mc_base"] != 0
    lo, hi = parse_size(args.min_size), parse_size(args.max_size)
    dnames = (args.datatype or args.dtypes or "bfloat16,float").split(",")
    tests = set(["on_stream", "barrier", "device"] if args.tests == "all" else args.tests.split(","))
    src = nv.tensor((hi,), torch.uint8)
    dst = nv.tensor((hi,), torch.uint8)
    src.random_(0, 100)
    lib = env.devlib()
    lib.perf_onstream_loop_algo.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=env.dev)
    flush = lambda: flush_buf.zero_()

    def iters_for(size):
        return args.iters if args.iters > 0 else (20 if size <= (16 << 20) else 8)

    def record(name, algo, dname, size, ms, how, factor_name, **extra):
        bw = size / (ms * 1e-3) / 1e9
        env.record(test=name, algo=algo, dtype=dname, bytes_per_pe=size, us=round(ms * 1e3, 2), algbw_GBps=round(bw, 2), busbw_GBps=round(bw * busbw_factor(factor_name, n), 2),
                   npes=n, nvls=nvls, issue=how, **extra)

    def run_ours(name, kind, algo_name, algo, dname, dcode, size, factor_name):
        """`iters` calls of one on-stream collective back to back: from a C loop (default) or replayed from a CUDA graph."""
        iters = iters_for(size)
        call = lambda k, st: ok(lib.perf_onstream_loop_algo(kind, C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), size, 0, k, algo, dcode, st))
        if args.cudagraph:
            ms, how = env.time_graph_ms(lambda st: call(1, C.c_void_p(st.cuda_stream)), iters=iters), "graph"
        else:
            call(args.warmup_iters, stream_ptr())
            ms, how = env.time_ms(lambda: call(iters, stream_ptr()), iters=1, warmup=0) / iters, "c-loop"
        extra = {}
        if size >= (8 << 20) and args.cold:
            extra["cold_us"] = round(env.time_ms(lambda: call(1, stream_ptr()), iters=5, warmup=1, flush=flush) * 1e3, 2)
        record(name, algo_name, dname, size, ms, how, factor_name, **extra)

    def pick(table, names):
        return ["auto"] if args.algos == "best" else [a for a in names if a in table] + ["auto"]

    if "on_stream" in tests:
        for dname in dnames:
            dt, dcode = DTYPES[dname]
            es = torch.empty((), dtype=dt).element_size()
            for size in sizes_geometric(lo, hi, args.step):
                cnt = size // es
                # allreduce: `size` bytes per PE
                for algo in pick(RED, ["oneshot", "twoshot"] + (["ll"] if size <= 2048 else []) + (["ll128"] if size <= 32768 else []) + (["nvls_oneshot", "nvls_twoshot"] if nvls else [])):
                    if algo in ("oneshot", "nvls_oneshot") and size > (4 << 20):
                        continue
                    run_ours("allreduce_on_stream", 0, algo, RED[algo], dname, dcode, size, "allreduce")
                if not args.no_nccl and n > 1:
                    t = torch.empty(cnt, dtype=dt, device=env.dev)
                    record("allreduce_nccl", "nccl", dname, size, env.time_ms(lambda: dist.all_reduce(t), iters=iters_for(size), warmup=3), "eager", "allreduce")
                # reducescatter / fcollect / alltoall: `size` bytes is the full buffer, size/n per block
                if cnt % n == 0 and cnt >= n:
                    blk = cnt // n
                    for algo in pick(RS, ["pull"] + (["nvls"] if nvls else [])):
                        run_ours("reducescatter_on_stream", 1, algo, RS[algo], dname, dcode, size, "reducescatter")
                    for algo in pick(FC, ["push"] + (["ll"] if size // n <= 2048 else []) + (["ll128"] if size // n <= 32768 else []) + (["nvls"] if nvls else [])):
                        run_ours("fcollect_on_stream", 2, algo, FC[algo], dname, dcode, size, "fcollect")
                    run_ours("alltoall_on_stream", 3, "push", 0, dname, dcode, size, "alltoall")
                    if not args.no_nccl and n > 1:
                        full, part = torch.empty(cnt, dtype=dt, device=env.dev), torch.empty(blk, dtype=dt, device=env.dev)
                        record("reducescatter_nccl", "nccl", dname, size, env.time_ms(lambda: dist.reduce_scatter_tensor(part, full), iters=iters_for(size), warmup=3), "eager", "reducescatter")
                        record("allgather_nccl", "nccl", dname, size, env.time_ms(lambda: dist.all_gather_into_tensor(full, part), iters=iters_for(size), warmup=3), "eager", "fcollect")
                        full2 = torch.empty(cnt, dtype=dt, device=env.dev)
                        record("alltoall_nccl", "nccl", dname, size, env.time_ms(lambda: dist.all_to_all_single(full2, full), iters=iters_for(size), warmup=3), "eager", "alltoall")
                for algo in pick(BC, ["push", "pull"] + (["ll"] if size <= 32768 else []) + (["nvls"] if nvls else [])):
                    run_ours("broadcast_on_stream", 4, algo, BC[algo], dname, dcode, size, "broadcast")
    # barrier / sync latency: on-stream (C loop and graph) and device-initiated at each scope
    if "barrier" in tests:
        lib.perf_onstream_loop.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
        for kind, name in ((5, "barrier_all_on_stream"), (6, "sync_all_on_stream")):
            ms = env.time_ms(lambda: ok(lib.perf_onstream_loop(kind, None, None, 0, 0, 100, stream_ptr())), iters=3, warmup=1)
            env.record(test=name, us=round(ms * 1e3 / 100, 2), npes=n, issue="c-loop")
        ms = env.time_graph_ms(lambda st: nv.barrier_all(stream=st), iters=50)
        env.record(test="barrier_all_on_stream", us=round(ms * 1e3, 2), npes=n, issue="graph")
        ms = env.time_graph_ms(lambda st: nv.sync_all(stream=st), iters=50)
        env.record(test="sync_all_on_stream", us=round(ms * 1e3, 2), npes=n, issue="graph")
        for scope, sname in scopes_of(args.scope):
            for sync_only in (0, 1):
                iters = 200
                ms = env.time_ms(lambda: ok(lib.perf_barrier_latency(iters, scope, sync_only, 256, stream_ptr())), iters=3, warmup=1)
                env.record(test="sync_device" if sync_only else "barrier_device", scope=sname, us=round(ms * 1e3 / iters, 3), npes=n)
    # device-initiated collectives at every scope, `iters` calls per launch
    if "device" in tests:
        lib.perf_coll_latency_scoped.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p]
        fsrc, fdst = src.view(torch.float32), dst.view(torch.float32)
        kinds = ((0, "allreduce_device_float", "allreduce", 4), (6, "allreduce_device_bfloat16", "allreduce", 2), (2, "reducescatter_device_float", "reducescatter", 4),
                 (3, "fcollect_device_int", "fcollect", 4), (4, "alltoall_device_int", "alltoall", 4), (5, "broadcast_device_int", "broadcast", 4))
        for kind, kname, fac, es in kinds:
            for scope, sname in scopes_of(args.scope):
                for size in sizes_geometric(max(lo, 64), min(hi, 4 << 20), max(args.step, 4)):
                    cnt = size // es
                    nel = cnt // n if kind in (2, 3, 4) else cnt
                    if nel < 1 or (scope != 2 and size > (256 << 10)):
                        continue  # one thread or one warp moving megabytes measures nothing of interest
                    iters = 50 if size <= 262144 else 10
                    ms = env.time_ms(lambda: ok(lib.perf_coll_latency_scoped(kind, C.c_void_p(fdst.data_ptr()), C.c_void_p(fsrc.data_ptr()), C.c_size_t(nel), iters, scope,
                                                                             1024 if scope == 2 else 32, stream_ptr())), iters=3, warmup=1)
                    us = ms * 1e3 / iters
                    env.record(test=kname, scope=sname, bytes=cnt * es, us=round(us, 2), busbw_GBps=round(cnt * es / (us * 1e-6) / 1e9 * busbw_factor(fac, n), 2), npes=n)
        ms = env.time_ms(lambda: ok(lib.perf_coll_latency_scoped(7, C.c_void_p(fdst.data_ptr()), C.c_void_p(fsrc.data_ptr()), C.c_size_t(1), 100, 2, 256, stream_ptr())), iters=3, warmup=1)
        env.record(test="redmaxloc_device_double2", scope="block", us=round(ms * 1e3 / 100, 2), npes=n)
    env.barrier()
    nv.free_tensor(src)
    nv.free_tensor(dst)
    env.finish()


if __name__ == "__main__":
    main()
