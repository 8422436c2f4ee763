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


def parse_size(s) -> int:
    """8, 4K, 32M, 1G (binary multiples), as the reference's perftests take them."""
    s = str(s)
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].lower()]) if s[-1].lower() in mult else int(s)


def add_reference_args(ap, min_size, max_size, iters, warmup, ctas=32, threads=1024, step=2):
    """The argument set shared by the reference's perftests (perftest/common/utils.cu:889-1010), with this driver's
    defaults: -b/-e/-f message sizes, -n/-w iterations, -c/-t launch geometry, -d datatype, -o reduce op, -s scope,
    -a atomic op, --bidir, --cudagraph, --issue."""
    ap.add_argument("-b", "--min_size", "--min-bytes", dest="min_size", default=min_size, help="smallest message (bytes; k/m/g suffixes)")
    ap.add_argument("-e", "--max_size", "--max-bytes", dest="max_size", default=max_size, help="largest message")
    ap.add_argument("-f", "--step", type=int, default=step, help="factor between consecutive message sizes")
    ap.add_argument("-n", "--iters", type=int, default=iters, help="timed iterations per size")
    ap.add_argument("-w", "--warmup_iters", type=int, default=warmup, help="untimed iterations before them")
    ap.add_argument("-c", "--ctas", type=int, default=ctas)
    ap.add_argument("-t", "--threads_per_cta", "--threads", dest="threads", type=int, default=threads)
    ap.add_argument("-d", "--datatype", default=None, help="element type(s), comma separated (collectives: float, bfloat16, half, int ...)")
    ap.add_argument("-o", "--reduce_op", default="sum")
    ap.add_argument("-s", "--scope", default="all", help="thread, warp, block or all")
    ap.add_argument("-a", "--atomic_op", default="all")
    ap.add_argument("--bidir", action="store_true", help="both PEs of a pair send at the same time")
    ap.add_argument("--cudagraph", action="store_true", help="replay the on-stream calls from a CUDA graph instead of issuing them eagerly")
    ap.add_argument("--issue", default="on_stream", help="on_stream (default) or host: how host-initiated operations are issued")
    return ap


def sizes_geometric(lo: int, hi: int, step: int = 2):
    s = max(1, lo)
    while s <= hi:
        yield s
        s *= max(2, step)


def scopes_of(arg: str):
    names = {"thread": 0, "warp": 1, "block": 2}
    return [(names[a], a) for a in (["block", "warp", "thread"] if arg == "all" else arg.split(","))]


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
