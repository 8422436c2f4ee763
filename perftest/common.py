"""Shared pieces of the perftest drivers: start-up under torchrun, device-side timing (CUDA events,
max over ranks), bus-bandwidth factors and result printing (a table for people, JSON lines with
``--json``).  Bus-bandwidth factors follow the usual convention (reference: perftest/common/utils.cu:581-609):
allreduce 2(n-1)/n, broadcast 1, alltoall / fcollect / reducescatter (n-1)/n."""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


class Env:
    def __init__(self):
        import nvshmem_b200.core as nv
        self.nv = nv
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
            nv.init(device=self.local_rank, initializer_method="torch")
        else:
            nv.init(device=self.local_rank, uid=nv.get_unique_id(), rank=0, nranks=1)
        self.rows = []

    def devlib(self):
        from nvshmem_b200.bindings import host as H
        H.load()
        lib = C.CDLL(str(H.lib_path("libbshmem_devtest.so")))
        H.load().nvshmemx_b200_module_sync()  # the library was loaded after init: hand it the device state
        assert lib.perf_preload() == 0
        return lib

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_ms(self, fn, iters=20, warmup=5, flush=None):
        """Mean device time of fn() in ms (CUDA events on the current stream), max over ranks."""
        for _ in range(warmup):
            fn()
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        if flush is None:
            start.record()
            for _ in range(iters):
                fn()
            end.record()
            torch.cuda.synchronize()
            total = start.elapsed_time(end)
        else:
            for _ in range(iters):
                flush()
                start.record()
                fn()
                end.record()
                torch.cuda.synchronize()
                total += start.elapsed_time(end)
        t = torch.tensor([total / iters], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_graph_ms(self, fn, iters=20):
        """Mean device time of one fn(stream) call in ms when `iters` calls are captured into a CUDA graph and
        replayed back to back: no host time between launches (the way the reference's C loops issue them)."""
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            fn(stream)  # warm-up outside the capture (module loading, lazy state)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(iters):
                    fn(stream)
        g.replay()
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        g.replay()
        end.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(end) / iters], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del g
        return float(t.item())

    def record(self, **row):
        self.rows.append(row)
        if self.rank == 0:
            print(json.dumps(row), flush=True)

    def finish(self):
        self.barrier()
        self.nv.finalize()
        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


def busbw_factor(coll: str, n: int) -> float:
    if n <= 1:
        return 1.0
    return {"reduce": 2.0 * (n - 1) / n, "allreduce": 2.0 * (n - 1) / n, "broadcast": 1.0}.get(coll, (n - 1) / n)


def sizes_pow2(lo: int, hi: int):
    s = lo
    while s <= hi:
        yield s
        s *= 2


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ok(rc: int) -> None:
    """Kernel launchers of the test library return non-zero when the launch failed."""
    if rc != 0:
        raise RuntimeError("kernel launch failed")
