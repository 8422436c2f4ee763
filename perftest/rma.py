"""Device-initiated RMA: put/get bandwidth at thread, warp and block scope, plain-store bandwidth, blocking latency,
put_signal and signal ping-pong latency, small-message rate, and the thirteen atomic operations (throughput and a
dependent-chain latency).  Every PE talks to its right neighbour (with two PEs: 0 <-> 1, i.e. both directions at once
for --bidir; without it only the even PEs send).

With no arguments the sweep is 8 B - 1 GB in powers of two, 1000 timed operations after 100 warm-up operations,
32 CTAs x 1024 threads, all three scopes.  The argument set is the reference's (-b -e -f -n -w -c -t -s -a --bidir).

  torchrun --nproc-per-node 2 -m perftest.rma [-b 8 -e 1G -n 1000 -w 100 -c 32 -t 1024 -s all]
(reference counterparts: perftest/device/pt-to-pt/shmem_{put,get}_bw, shmem_st_bw, shmem_{put,get}_latency,
 shmem_put_signal_ping_pong_latency, shmem_signal_ping_pong_latency, shmem_{p,g}_bw, shmem_atomic_{bw,latency})
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from .common import Env, add_reference_args, ok, parse_size, scopes_of, sizes_geometric, stream_ptr  # noqa: F401

ATOMICS = ["fetch_add", "add", "compare_swap", "swap", "fetch_or", "inc", "fetch_inc", "and", "fetch_and", "or", "xor", "fetch_xor", "set"]


def main():
    ap = argparse.ArgumentParser()
    add_reference_args(ap, min_size="8", max_size="1G", iters=1000, warmup=100, ctas=32, threads=1024)
    ap.add_argument("--tests", default="all", help="comma list of: bw, st_bw, latency, pingpong, rate, atomics")
    args = ap.parse_args()
    env = Env()
    nv, lib = env.nv, env.devlib()
    n, me = env.world, env.rank
    right = (me + 1) % n
    max_bytes, min_bytes = parse_size(args.max_size), parse_size(args.min_size)
    tests = set(["bw", "st_bw", "latency", "pingpong", "rate", "atomics"] if args.tests == "all" else args.tests.split(","))
    sym = nv.tensor((max(max_bytes, 1 << 20),), torch.uint8)
    local = torch.empty(max(max_bytes, 1 << 20), dtype=torch.uint8, device=env.dev)
    counter = torch.zeros(1, dtype=torch.int32, device=env.dev)
    sink = torch.zeros(4, dtype=torch.int64, device=env.dev)
    sends = args.bidir or n != 2 or me == 0  # two PEs without --bidir: one direction, as in the reference

    def timed(call, iters, warmup):
        """One launch of `warmup` operations (untimed), then one launch of `iters` timed with CUDA events; max over ranks."""
        if warmup:
            call(warmup)
        return env.time_ms(lambda: call(iters), iters=1, warmup=0)

    # ---- bandwidth
    if "bw" in tests:
        for direction, dname in ((0, "put"), (1, "get")):
            for scope, sname in scopes_of(args.scope):
                for size in sizes_geometric(max(min_bytes, 16), max_bytes, args.step):
                    ctas = max(1, min(args.ctas, size // 4096))
                    def call(k):
                        if sends:
                            ok(lib.perf_bw(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), right, k, scope, direction, ctas, args.threads,
                                           C.c_void_p(counter.data_ptr()), stream_ptr()))
                    ms = timed(call, args.iters, args.warmup_iters)
                    moved = (size // ctas // 16 * 16) * ctas
                    env.record(test=f"{dname}_bw", scope=sname, bytes=size, ctas=ctas, iters=args.iters, us=round(ms * 1e3 / args.iters, 3),
                               GBps=round(moved * args.iters / (ms * 1e-3) / 1e9, 2), npes=n, bidir=bool(args.bidir))
    if "st_bw" in tests:
        lib.perf_st_bw.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        for size in sizes_geometric(max(min_bytes, 1024), max_bytes, args.step):
            ctas = max(1, min(args.ctas, size // 8192))
            def call(k):
                if sends:
                    ok(lib.perf_st_bw(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), size, right, k, ctas, args.threads, C.c_void_p(counter.data_ptr()), stream_ptr()))
            ms = timed(call, args.iters, args.warmup_iters)
            env.record(test="st_bw", bytes=size, ctas=ctas, iters=args.iters, us=round(ms * 1e3 / args.iters, 3), GBps=round(size * args.iters / (ms * 1e-3) / 1e9, 2), npes=n)
    # ---- blocking latency (one group, put + quiet / get); the get chain reads its next offset from the data, which is zero
    if "latency" in tests:
        sym.zero_()
        local.zero_()
        env.barrier()
        for dname, fn in (("put_latency", lib.perf_put_latency), ("get_latency", lib.perf_get_latency)):
            for scope, sname in scopes_of(args.scope):
                for size in sizes_geometric(min_bytes, min(max_bytes, 1 << 20), args.step):
                    iters = args.iters if size <= 65536 else max(20, args.iters // 10)
                    def call(k):
                        ok(fn(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), right, k, scope, 1024 if scope == 2 else 32, stream_ptr()))
                    ms = timed(call, iters, max(1, args.warmup_iters // 10))
                    env.record(test=dname, scope=sname, bytes=size, iters=iters, us=round(ms * 1e3 / iters, 3), npes=n)
    # ---- ping-pong (PE 0 <-> PE 1)
    if "pingpong" in tests and n >= 2:
        sig = nv.tensor((2,), torch.int64, zero=True)
        base = [0]
        for scope, sname in scopes_of(args.scope):
            for size in sizes_geometric(min_bytes, min(max_bytes, 1 << 20), args.step):
                iters = min(args.iters, 500)
                def call(k):
                    ok(lib.perf_pingpong(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), C.c_void_p(sig.data_ptr()), k, C.c_uint64(base[0]), scope,
                                         1024 if scope == 2 else 32, stream_ptr()))
                    base[0] += k
                ms = timed(call, iters, 20)
                env.record(test="put_signal_pingpong", scope=sname, bytes=size, iters=iters, us_round_trip=round(ms * 1e3 / iters, 3), us_one_way=round(ms * 1e3 / iters / 2, 3), npes=n)
        def call2(k):
            ok(lib.perf_signal_pingpong(C.c_void_p(sig.data_ptr()), k, C.c_uint64(base[0]), stream_ptr()))
            base[0] += k
        ms = timed(call2, 1000, 100)
        env.record(test="signal_pingpong", iters=1000, us_round_trip=round(ms * 1e3 / 1000, 3), us_one_way=round(ms * 1e3 / 1000 / 2, 3), npes=n)
        env.barrier()
        nv.free_tensor(sig)
    # ---- small-message rate and atomics
    words = nv.tensor((args.ctas * 1024,), torch.int64, zero=True)
    if "rate" in tests:
        for direction, dname in ((0, "p_rate"), (1, "g_rate")):
            iters = min(args.iters, 1000)
            def call(k):
                ok(lib.perf_pg_rate(C.c_void_p(words.data_ptr()), right, k, direction, args.ctas, 1024, C.c_void_p(sink.data_ptr()), stream_ptr()))
            ms = timed(call, iters, args.warmup_iters)
            ops = iters * args.ctas * 1024
            env.record(test=dname, iters=iters, Mops=round(ops / (ms * 1e-3) / 1e6, 1), GBps=round(ops * 8 / (ms * 1e-3) / 1e9, 2), npes=n)
    if "atomics" in tests:
        wanted = ATOMICS if args.atomic_op == "all" else args.atomic_op.split(",")
        for kname in wanted:
            kind = ATOMICS.index(kname)
            for contend in (0, 1):
                iters = min(args.iters, 500)
                def call(k):
                    ok(lib.perf_atomic_rate(C.c_void_p(words.data_ptr()), right, k, kind, contend, args.ctas, 256, C.c_void_p(sink.data_ptr()), stream_ptr()))
                ms = timed(call, iters, max(1, args.warmup_iters // 2))
                ops = iters * args.ctas * 256
                env.record(test=f"atomic_{kname}", contended=bool(contend), iters=iters, Mops=round(ops / (ms * 1e-3) / 1e6, 1), us_per_op_per_thread=round(ms * 1e3 / iters, 4),
                           npes=n, dtype="int64")
        def call3(k):
            ok(lib.perf_atomic_latency(C.c_void_p(words.data_ptr()), right, k, C.c_void_p(sink.data_ptr()), stream_ptr()))
        ms = timed(call3, 1000, 100)
        env.record(test="atomic_fetch_add_latency", iters=1000, us=round(ms * 1e3 / 1000, 3), npes=n, note="dependent chain of one thread: one link round trip per operation")
    env.barrier()
    nv.free_tensor(words)
    nv.free_tensor(sym)
    env.finish()


if __name__ == "__main__":
    main()
