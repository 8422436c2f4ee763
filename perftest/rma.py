"""Device-initiated RMA: put/get bandwidth at thread, warp and block scope, blocking latency,
put_signal and signal ping-pong latency, small-message rate and atomic throughput / latency.
PE 0 talks to PE 1 (and, with more PEs, every PE to its right neighbour for the bandwidth rows).

  torchrun --nproc-per-node 2 -m perftest.rma [--max-bytes 1G] [--iters 20]
(reference counterparts: perftest/device/pt-to-pt/shmem_{put,get}_bw, shmem_{put,get}_latency,
 shmem_put_signal_ping_pong_latency, shmem_signal_ping_pong_latency, shmem_{p,g}_bw, shmem_atomic_{bw,latency})
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from .common import Env, sizes_pow2, stream_ptr, ok


def parse_size(s: str) -> int:
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].lower()]) if s[-1].lower() in mult else int(s)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--min-bytes", default="8")
    ap.add_argument("--iters", type=int, default=10, help="operations per kernel launch")
    ap.add_argument("--ctas", type=int, default=32)
    ap.add_argument("--threads", type=int, default=1024)
    args = ap.parse_args()
    env = Env()
    nv, lib = env.nv, env.devlib()
    n, me = env.world, env.rank
    right = (me + 1) % n
    max_bytes, min_bytes = parse_size(args.max_bytes), parse_size(args.min_bytes)
    sym = nv.tensor((max_bytes,), torch.uint8)
    local = torch.empty(max_bytes, dtype=torch.uint8, device=env.dev)
    counter = torch.zeros(1, dtype=torch.int32, device=env.dev)
    sink = torch.zeros(4, dtype=torch.int64, device=env.dev)
    scope_name = {0: "thread", 1: "warp", 2: "block"}

    # ---- bandwidth
    for direction, dname in ((0, "put"), (1, "get")):
        for scope in (2, 1, 0):
            for size in sizes_pow2(max(min_bytes, 1 << 10), max_bytes):
                ctas = max(1, min(args.ctas, size // 4096))
                iters = args.iters if size <= (64 << 20) else max(2, args.iters // 4)
                fn = lambda: ok(lib.perf_bw(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), right, iters, scope, direction, ctas, args.threads,
                                         C.c_void_p(counter.data_ptr()), stream_ptr()))
                ms = env.time_ms(fn, iters=5, warmup=2)
                moved = (size // ctas // 16 * 16) * ctas
                env.record(test=f"{dname}_bw", scope=scope_name[scope], bytes=size, ctas=ctas, us=round(ms * 1e3 / iters, 3), GBps=round(moved * iters / (ms * 1e-3) / 1e9, 2), npes=n)
    # ---- blocking latency (one group, put + quiet / get); the get chain reads its next offset from the data, which is zero
    sym.zero_()
    local.zero_()
    env.barrier()
    for dname, call in (("put_latency", lib.perf_put_latency), ("get_latency", lib.perf_get_latency)):
        for scope in (0, 1, 2):
            for size in sizes_pow2(min_bytes, min(max_bytes, 1 << 20)):
                iters = 200 if size <= 65536 else 20
                fn = lambda: ok(call(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), right, iters, scope, 1024 if scope == 2 else 32, stream_ptr()))
                ms = env.time_ms(fn, iters=3, warmup=1)
                env.record(test=dname, scope=scope_name[scope], bytes=size, us=round(ms * 1e3 / iters, 3), npes=n)
    # ---- ping-pong (PE 0 <-> PE 1)
    if n >= 2:
        sig = nv.tensor((2,), torch.int64, zero=True)
        base = 0
        for scope in (0, 1, 2):
            for size in sizes_pow2(min_bytes, min(max_bytes, 1 << 20)):
                iters = 200
                def fn():
                    nonlocal base
                    ok(lib.perf_pingpong(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), C.c_void_p(sig.data_ptr()), iters, C.c_uint64(base), scope,
                                      1024 if scope == 2 else 32, stream_ptr()))
                    base += iters
                ms = env.time_ms(fn, iters=3, warmup=1)
                env.record(test="put_signal_pingpong", scope=scope_name[scope], bytes=size, us_one_way=round(ms * 1e3 / iters / 2, 3), npes=n)
        def fn2():
            nonlocal base
            ok(lib.perf_signal_pingpong(C.c_void_p(sig.data_ptr()), 500, C.c_uint64(base), stream_ptr()))
            base += 500
        ms = env.time_ms(fn2, iters=3, warmup=1)
        env.record(test="signal_pingpong", us_one_way=round(ms * 1e3 / 500 / 2, 3), npes=n)
        env.barrier()
        nv.free_tensor(sig)
    # ---- small-message rate and atomics
    words = nv.tensor((args.ctas * 1024,), torch.int64, zero=True)
    for direction, dname in ((0, "p_rate"), (1, "g_rate")):
        iters = 200
        fn = lambda: ok(lib.perf_pg_rate(C.c_void_p(words.data_ptr()), right, iters, direction, args.ctas, 1024, C.c_void_p(sink.data_ptr()), stream_ptr()))
        ms = env.time_ms(fn, iters=3, warmup=1)
        ops = iters * args.ctas * 1024
        env.record(test=dname, Mops=round(ops / (ms * 1e-3) / 1e6, 1), GBps=round(ops * 8 / (ms * 1e-3) / 1e9, 2), npes=n)
    for kind, kname in ((0, "fetch_add"), (1, "add"), (2, "compare_swap"), (3, "swap"), (4, "fetch_or")):
        for contend in (0, 1):
            iters = 100
            fn = lambda: ok(lib.perf_atomic_rate(C.c_void_p(words.data_ptr()), right, iters, kind, contend, args.ctas, 256, C.c_void_p(sink.data_ptr()), stream_ptr()))
            ms = env.time_ms(fn, iters=3, warmup=1)
            env.record(test=f"atomic_{kname}", contended=bool(contend), Mops=round(iters * args.ctas * 256 / (ms * 1e-3) / 1e6, 1), npes=n)
    fn = lambda: ok(lib.perf_atomic_latency(C.c_void_p(words.data_ptr()), right, 500, C.c_void_p(sink.data_ptr()), stream_ptr()))
    ms = env.time_ms(fn, iters=3, warmup=1)
    env.record(test="atomic_fetch_add_latency", us=round(ms * 1e3 / 500, 3), npes=n)
    env.barrier()
    nv.free_tensor(words)
    nv.free_tensor(sym)
    env.finish()


if __name__ == "__main__":
    main()
