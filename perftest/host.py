"""Host-initiated paths: put/get bandwidth and latency (blocking, non-blocking + quiet, on-stream),
stream-ordered signal round trip and symmetric allocation time against size.

  torchrun --nproc-per-node 2 -m perftest.host
(reference counterparts: perftest/host/pt-to-pt/{bw,latency,stream_latency}, perftest/host/init/malloc)
"""
from __future__ import annotations

import argparse
import ctypes as C
import time

import torch

from .common import Env, ok, sizes_pow2, stream_ptr
from .common import parse_size


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--malloc-max", default="8G")
    args = ap.parse_args()
    env = Env()
    nv, n = env.nv, env.world
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    right = (env.rank + 1) % n
    hi = parse_size(args.max_bytes)
    sym = nv.tensor((hi,), torch.uint8)
    local = torch.empty(hi, dtype=torch.uint8, device=env.dev)
    try:
        dev = env.devlib()
        dev.perf_onstream_loop.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    except (OSError, AssertionError):
        dev = None
    for size in sizes_pow2(8, hi):
        iters = 20 if size <= (1 << 20) else 5
        for name, fn in (("host_put_on_stream", lambda: lib.nvshmemx_putmem_on_stream(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), size, right, stream_ptr())),
                         ("host_get_on_stream", lambda: lib.nvshmemx_getmem_on_stream(C.c_void_p(local.data_ptr()), C.c_void_p(sym.data_ptr()), size, right, stream_ptr()))):
            ms = env.time_ms(fn, iters=iters, warmup=2)
            env.record(test=name, bytes=size, us=round(ms * 1e3, 2), GBps=round(size / (ms * 1e-3) / 1e9, 2), npes=n)
        if dev is not None:
            # the same calls issued from a C loop (no interpreter between them), as the reference's host perftests do
            for kind, name, d, sbuf in ((7, "host_put_on_stream", sym, local), (8, "host_get_on_stream", local, sym)):
                reps = 50
                ms = env.time_ms(lambda: ok(dev.perf_onstream_loop(kind, C.c_void_p(d.data_ptr()), C.c_void_p(sbuf.data_ptr()), size, right, reps, stream_ptr())), iters=3, warmup=1)
                env.record(test=name, bytes=size, us=round(ms * 1e3 / reps, 2), GBps=round(size / (ms * 1e-3 / reps) / 1e9, 2), npes=n, issue="c-loop")
        t0 = time.perf_counter()
        for _ in range(iters):
            lib.nvshmem_putmem(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), size, right)
        dt = (time.perf_counter() - t0) / iters
        env.record(test="host_put_blocking_wallclock", bytes=size, us=round(dt * 1e6, 2), GBps=round(size / dt / 1e9, 2), npes=n)
    # stream-ordered signal round trip with the right neighbour
    sig = nv.tensor((1,), torch.int64, zero=True)
    env.barrier()
    val = [0]
    def sigstep():
        val[0] += 1
        nv.signal_op(sig, val[0], nv.SignalOp.SIGNAL_SET, right)
        nv.signal_wait(sig, val[0], nv.ComparisonType.CMP_GE)
    ms = env.time_ms(sigstep, iters=50, warmup=5)
    env.record(test="stream_signal_set_and_wait", us=round(ms * 1e3, 2), npes=n)
    env.barrier()
    nv.free_tensor(sig)
    nv.free_tensor(sym)
    # allocation time against size (collective: includes growth, handle exchange and the barrier)
    size = 1 << 20
    top = parse_size(args.malloc_max)
    while size <= top:
        env.barrier()
        t0 = time.perf_counter()
        p = lib.nvshmem_malloc(size)
        dt = time.perf_counter() - t0
        t1 = time.perf_counter()
        lib.nvshmem_free(C.c_void_p(p))
        df = time.perf_counter() - t1
        env.record(test="nvshmem_malloc", bytes=size, malloc_ms=round(dt * 1e3, 3), free_ms=round(df * 1e3, 3), heap_chunks=nv.heap_info()["chunks"], npes=n)
        size *= 4
    env.finish()


if __name__ == "__main__":
    main()
