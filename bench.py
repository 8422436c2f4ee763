#!/usr/bin/env python
"""Headline benchmark: row-parallel GEMM fused with reduce-scatter (config (d) of the work list).

Per rank: x[M=8192, K=3584] @ w[N=8192, K=3584]^T in bf16 with fp32 accumulation, summed over the
ranks and scattered by rows (weak scaling: the K-slice per rank is fixed, so per-GPU work is
constant).  The metric is the whole-job TFLOP/s = n_gpus * 2*M*N*K / step time.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--repeats R] [--layers L]

For N > 1 launch with torchrun (one rank per GPU); rank 0 prints one JSON line.

Device-timed value: CUDA events on the launching stream around exactly K steps, barrier +
synchronize on both sides, max over ranks; that region is repeated R times in the same process and
the median region is reported (all regions are listed under `repeats`), so that the number is a
steady-state one.  Inputs rotate through several buffer sets whose total size exceeds the 126 MB L2.
SM clocks and throttle reasons are sampled through NVML over all regions.

End-to-end value (`e2e`): the same GEMM shapes as a unit of model work through the public API, a
stack of L tensor-parallel MLP blocks (all-gather -> GEMM + GELU, GEMM -> reduce-scatter; hidden
8192, 3584 FFN columns per rank, 8192 tokens).  Every step copies this rank's token shard from
pinned host memory to the device, runs the L blocks, and copies the rank's output shard back to
pinned host memory; copies of neighbouring steps overlap the compute on side streams, and the timed
region ends when the last result is on the host.  Its TFLOP/s counts the 2 L GEMMs of a step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

M, N, K_LOCAL = 8192, 8192, 3584
HIDDEN = N            # MLP stack of the end-to-end run: hidden size = N, FFN columns per rank = K_LOCAL
BASELINE_VALUE = None  # the reference publishes no number for this metric


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sets", type=int, default=3, help="input buffer sets rotated between steps")
    ap.add_argument("--repeats", type=int, default=10, help="how many times the timed region of --steps steps is run (median reported)")
    ap.add_argument("--layers", type=int, default=8, help="MLP blocks per step of the end-to-end run")
    ap.add_argument("--e2e-repeats", type=int, default=3)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only queries) from a
    thread while a region runs."""

    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.sm, self.power, self.reasons = [], [], set()
        self.sm_max = None
        self._stop = threading.Event()
        self.thread = None

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["NVML unavailable"]}
        self._stop.set()
        self.thread.join(timeout=2)
        # "under load": samples taken while the GPU drew more than half of the highest power seen
        loaded = [c for c, p in zip(self.sm, self.power) if self.power and p >= 0.5 * max(self.power)]
        return {"sm_mhz": statistics.median(loaded or self.sm) if self.sm else None, "sm_max_mhz": self.sm_max, "samples": len(self.sm),
                "samples_under_load": len(loaded), "power_w_max": round(max(self.power), 1) if self.power else None, "reasons": sorted(self.reasons)}


def reference_arm(args):
    """Runs the unmodified reference build (baseline/_ref) for the same metric: cuBLAS GEMM
    (torch.matmul) followed by the reference library's own bf16 sum reducescatter on the stream."""
    from baseline import reference_bench
    return reference_bench.run(args, M, N, K_LOCAL)


def timed_runs(step, stack, args, M, N, K_LOCAL, rank, world, local_rank, launches_per_step, errors=None):
    """Times `step(x, w) -> out` on device-resident inputs (R regions of --steps steps), then the end-to-end run of
    `stack` (an object with `input_shard`, `forward(out_index) -> tensor`, `kernels_per_forward`).  Returns the JSON
    line (without `impl`).  Both arms of the benchmark go through this function.  `errors()`, when given, returns a
    description of what went wrong on the device since its last call, or None (collective over the ranks)."""
    import torch
    import torch.distributed as dist

    dev = torch.device("cuda", local_rank)
    torch.manual_seed(1234 + rank)
    sets = max(1, args.sets)
    xs = [torch.randn(M, K_LOCAL, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(sets)]
    ws = [torch.randn(N, K_LOCAL, device=dev, dtype=torch.float32).mul_(0.02).to(torch.bfloat16) for _ in range(sets)]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    warm = max(3, args.warmup)
    for i in range(warm):
        step(xs[i % sets], ws[i % sets])
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    regions = []
    for r in range(max(1, args.repeats)):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(args.steps):
            step(xs[i % sets], ws[i % sets])
        end.record()
        barrier()
        regions.append(start.elapsed_time(end))
    regions = max_over_ranks(regions)               # per region: the slowest rank
    per_step = sorted(ms / args.steps for ms in regions)
    ms_per_step = statistics.median(per_step)
    flops_per_rank = 2.0 * M * N * K_LOCAL
    value = world * flops_per_rank / (ms_per_step * 1e-3) / 1e12
    del xs, ws
    device_timed_error = errors() if errors else None

    # ---------------- end to end: L MLP blocks per step, token shard in from pinned host memory, output shard back out
    rows = M // world
    host_in = [torch.randn(rows, HIDDEN, dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(2)]
    host_out = [torch.empty(rows, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_in = [torch.empty(rows, HIDDEN, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    in_stream, out_stream = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    h2d_done = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    fwd_done = [torch.cuda.Event() for _ in range(2)]
    d2h_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(n):
        for i in range(n):
            b = i & 1
            if i >= 2:
                d2h_done[b].synchronize()       # at most two steps in flight; step i-2's result is on the host
            with torch.cuda.stream(in_stream):  # host -> device copy of this step's tokens, ahead of the compute
                if i >= 2:
                    in_stream.wait_event(in_free[b])
                dev_in[b].copy_(host_in[b], non_blocking=True)
                h2d_done[b].record(in_stream)
            main.wait_event(h2d_done[b])
            stack.input_shard.copy_(dev_in[b], non_blocking=True)
            in_free[b].record(main)
            if i >= 2:
                main.wait_event(d2h_done[b])    # the output buffer of step i-2 has been read out
            out = stack.forward(b)
            fwd_done[b].record(main)
            with torch.cuda.stream(out_stream):  # device -> host copy of this step's result shard
                out_stream.wait_event(fwd_done[b])
                host_out[b].copy_(out, non_blocking=True)
                d2h_done[b].record(out_stream)
        main.wait_event(d2h_done[(n - 1) & 1])
        if n >= 2:
            main.wait_event(d2h_done[(n - 2) & 1])

    e2e_steps(max(3, min(args.warmup, 5)))
    barrier()
    e2e_regions = []
    for r in range(max(1, args.e2e_repeats)):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0.record()
        in_stream.wait_event(t0)
        e2e_steps(args.steps)
        t1.record()   # after the main stream has waited for the last device -> host copies
        barrier()
        e2e_regions.append(t0.elapsed_time(t1))
    clocks = sampler.stop()
    e2e_regions = max_over_ranks(e2e_regions)
    e2e_per_step = sorted(ms / args.steps for ms in e2e_regions)
    e2e_ms_per_step = statistics.median(e2e_per_step)
    L = stack.layers
    e2e_value = world * (2 * L * flops_per_rank) / (e2e_ms_per_step * 1e-3) / 1e12
    checksum = float(host_out[(args.steps - 1) & 1].float().abs().mean())
    e2e_error = errors() if errors else None
    line = {
        "metric": "fused_gemm_reduce_scatter_tflops",
        "value": round(value, 2),
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": warm,
        "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None,
        "dtype": "bf16",
        "data": "synthetic (seeded randn activations, N(0,0.02) weights, random init)",
        "config": {"model": "tp_row_parallel_gemm_reduce_scatter", "M": M, "N": N, "K_per_rank": K_LOCAL, "global_batch": M, "seq_len": 1,
                   "parallelism": f"tp{world}", "l2": f"inputs rotate over {sets} buffer sets ({sets * (M + N) * K_LOCAL * 2 >> 20} MiB > 126 MiB L2)",
                   "e2e_model": f"{L} x tp_mlp(hidden {HIDDEN}, ffn {K_LOCAL} per rank, {M} tokens): all-gather->GEMM+GELU, GEMM->reduce-scatter"},
        "repeats": {"regions": len(per_step), "ms_per_step_min": round(per_step[0], 5), "ms_per_step_median": round(ms_per_step, 5),
                    "ms_per_step_max": round(per_step[-1], 5)},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms_per_step, 5), "h2d_bytes_per_step": rows * HIDDEN * 2,
                "d2h_bytes_per_step": rows * HIDDEN * 2, "layers": L, "regions": len(e2e_per_step), "ms_per_step_min": round(e2e_per_step[0], 5),
                "ms_per_step_max": round(e2e_per_step[-1], 5), "gpu_launches": args.steps * len(e2e_per_step) * stack.kernels_per_forward,
                "output_abs_mean": round(checksum, 6)},
        "gpu_launches": args.steps * len(per_step) * launches_per_step,
    }
    if device_timed_error:
        line["invalid"] = device_timed_error
    if e2e_error:
        line["e2e"]["invalid"] = e2e_error
    return line


def main():
    args = parse()
    if args.impl == "reference":
        try:
            line = reference_arm(args)
        except Exception as e:  # the reference arm must never take the driver down
            line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(line), flush=True)
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    # The benchmark's buffers (two generations of partial tiles, the gathered activations) are backed at start-up.
    os.environ.setdefault("NVSHMEM_SYMMETRIC_SIZE", "2G")
    import nvshmem_b200.core as nv
    from nvshmem_b200.models.tp_mlp import TensorParallelMLPStack
    from nvshmem_b200.ops import fused_gemm as fg

    if world > 1:
        nv.init(device=local_rank, initializer_method="torch")
    else:
        nv.init(device=local_rank, uid=nv.get_unique_id(), rank=0, nranks=1)
    op = fg.GemmReduceScatter(M, N, mode="rs")

    class Stack:
        """The public model object behind the interface the timing harness wants."""

        def __init__(self, gather):
            self.model = TensorParallelMLPStack(HIDDEN, K_LOCAL * world, M, args.layers, seed=99 + rank, gather=gather, wait_limit_ms=3000)
            self.layers = args.layers
            self.kernels_per_forward = self.model.kernels_per_forward
            self.outs = [torch.empty_like(self.model.out) for _ in range(2)]
            self.input_shard = self.model.input_shard

        def forward(self, b):
            self.model.out = self.outs[b]
            return self.model.forward()

    def errors():
        bad = torch.tensor([fg.take_error(dev)], device=dev, dtype=torch.int32)
        if world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        return "a kernel gave up on a bounded wait" if int(bad.item()) else None

    def works(stack):
        """Two forward passes; true when no kernel of any rank gave up on a wait (the waits are bounded: a path that
        does not work on this machine costs seconds, not the run)."""
        for b in range(2):
            stack.forward(b)
        return errors() is None

    stack = Stack("fused")
    e2e_path = "all-gather fused into the GEMM kernel"
    if not works(stack):
        stack.model.close()
        stack = Stack("collective")
        e2e_path = "all-gather by the library's fcollect kernel, then the GEMM kernel (the fused all-gather gave up on a wait in the trial passes)"
        if not works(stack):
            e2e_path += "; this path gave up on a wait as well: the end-to-end figure is not valid"
    # one fused tcgen05 kernel per step (libbshmem_fused.so): GEMM, partial tiles, flags and the reduction
    line = timed_runs(lambda x, w: op(x, w), stack, args, M, N, K_LOCAL, rank, world, local_rank, launches_per_step=1, errors=errors)
    line["impl"] = "ours"
    line["e2e"]["path"] = e2e_path
    line["path"] = "one fused kernel per step; partial tiles reduced by " + ("the switch (multimem.ld_reduce)" if op.switch_path else ("pushes to the owner" if world > 1 else "nobody (one PE)"))
    stack.model.close()
    op.close()
    nv.finalize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
