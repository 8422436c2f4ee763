"""Small single-GPU cases of each hand-written kernel, sized for a profiler capture (inputs larger than
the 126 MB L2 where DRAM figures matter, a few hundred MB on the device at most, a handful of launches).

  python -m perftest.kernel_case --kernel gemm            # tcgen05 GEMM, 4096 x 4096 x 4096
  python -m perftest.kernel_case --kernel gemm_bench      # the benchmark shape 8192 x 8192 x 3584
  python -m perftest.kernel_case --kernel moe_dispatch    # one-PE dispatch, 4096 tokens x 7168, top-8 of 256
  python -m perftest.kernel_case --kernel moe_dispatch_fp8
  python -m perftest.kernel_case --kernel moe_combine
  python -m perftest.kernel_case --kernel allreduce       # one-PE on-stream allreduce kernel (copy path)
Prints the CUDA-event time of the last launch.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def timed(fn, launches: int):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ms = 0.0
    for _ in range(launches):
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm")
    ap.add_argument("--launches", type=int, default=4)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    from nvshmem_b200.ops import fused_gemm as fg
    if args.kernel in ("gemm", "gemm_bench"):
        M, N, K = (4096, 4096, 4096) if args.kernel == "gemm" else (8192, 8192, 3584)
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms = timed(lambda: fg.gemm(x, w, out), args.launches)
        print(f"{args.kernel}: {ms:.4f} ms, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
        fg.check_errors()
        return
    import nvshmem_b200.core as nv
    nv.init(device=0, uid=nv.get_unique_id(), rank=0, nranks=1)
    try:
        if args.kernel.startswith("moe"):
            from nvshmem_b200.ops.moe import MoeDispatchCombine
            T, H, K, E = 4096, 7168, 8, 256
            x = torch.randn(T, H, device=dev).to(torch.bfloat16)
            w, idx = torch.randn(T, E, device=dev).softmax(-1).topk(K, dim=-1)
            idx, w = idx.to(torch.int32).contiguous(), w.float().contiguous()
            moe = MoeDispatchCombine(T, H, K, E, payload="fp8" if args.kernel.endswith("fp8") else "bf16")
            ms = timed(lambda: moe.dispatch(x, idx), args.launches)
            row = H + H // 32 if args.kernel.endswith("fp8") else 2 * H
            print(f"moe dispatch: {ms * 1e3:.1f} us, reads {T * H * 2 / 1e6:.0f} MB, writes {T * K * row / 1e6:.0f} MB, {(T * H * 2 + T * K * row) / ms / 1e6:.0f} GB/s")
            if args.kernel == "moe_combine":
                rows = int(moe.expert_offsets[-1])
                moe.expert_out[:rows] = moe.recv_x[:rows]
                ms = timed(lambda: moe.combine(idx, w), args.launches)
                print(f"moe combine: {ms * 1e3:.1f} us, reads {T * K * H * 2 / 1e6:.0f} MB, writes {T * H * 2 / 1e6:.0f} MB, {(T * K + T) * H * 2 / ms / 1e6:.0f} GB/s")
            fg.check_errors()
            moe.close()
        elif args.kernel == "allreduce":
            n = 64 << 20
            src, dst = nv.tensor((n,), torch.float32), nv.tensor((n,), torch.float32)
            src.fill_(1.0)
            ms = timed(lambda: nv.reduce(0, dst, src, "sum"), args.launches)
            print(f"allreduce (1 PE, copy path): {ms * 1e3:.1f} us, {2 * n * 4 / ms / 1e6:.0f} GB/s")
        else:
            raise SystemExit(f"unknown kernel {args.kernel}")
    finally:
        nv.finalize()


if __name__ == "__main__":
    main()
