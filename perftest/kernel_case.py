"""Small single-GPU cases of each hand-written kernel, sized for a profiler capture (inputs larger than
the 126 MB L2 where DRAM figures matter, a few hundred MB on the device at most, a handful of launches).

  python -m perftest.kernel_case --kernel gemm            # tcgen05 GEMM, 4096 x 4096 x 4096
  python -m perftest.kernel_case --kernel gemm_bench      # the benchmark shape 8192 x 8192 x 3584
  python -m perftest.kernel_case --kernel moe_dispatch    # one-PE dispatch, 4096 tokens x 7168, top-8 of 256
  python -m perftest.kernel_case --kernel moe_dispatch_fp8
  python -m perftest.kernel_case --kernel moe_combine
  python -m perftest.kernel_case --kernel allreduce       # one-PE on-stream allreduce kernel (copy path)
  python -m perftest.kernel_case --kernel reducescatter | fcollect | alltoall | broadcast   # the other on-stream kernels, one PE
  python -m perftest.kernel_case --kernel put_bw          # block-scope put loop of the RMA perftest onto this PE's own heap
  python -m perftest.kernel_case --kernel get_bw
  python -m perftest.kernel_case --kernel grouped_gemm    # grouped tcgen05 GEMM with the gated activation, 32 ragged groups
  BSHMEM_FUSED_2CTA=0 python -m perftest.kernel_case --kernel gemm   # the one-CTA-per-tile variant of the GEMM kernel
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
    if args.kernel == "grouped_gemm":
        G, N, K, R = 32, 4096, 7168, 16384   # 32 experts, gate + up of 2048 each, 16384 routed rows in ragged groups
        sizes = torch.full((G,), R // G, dtype=torch.int64)
        sizes[::2] += 37
        sizes[1::2] -= 37
        offs = torch.zeros(G + 1, dtype=torch.int32)
        offs[1:] = sizes.cumsum(0).to(torch.int32)
        x = torch.randn(R, K, device=dev).to(torch.bfloat16)
        w = fg.interleave_gate_up((torch.randn(G, N, K, device=dev) * 0.02).to(torch.bfloat16))
        out = torch.empty(R, N // 2, device=dev, dtype=torch.bfloat16)
        offs_d = offs.to(dev)
        ms = timed(lambda: fg.grouped_gemm(x, w, offs_d, out=out, act="swiglu"), args.launches)
        print(f"grouped_gemm: {ms:.4f} ms, {2 * R * N * K / ms / 1e9:.1f} TFLOP/s ({G} groups, rows {int(sizes.min())}-{int(sizes.max())})")
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
        elif args.kernel in ("reducescatter", "fcollect", "alltoall", "broadcast"):
            n = 64 << 20
            src, dst = nv.tensor((n,), torch.float32), nv.tensor((n,), torch.float32)
            src.fill_(1.0)
            ms = timed(lambda: nv.collective_on_buffer(args.kernel, 0, dst, src, op="sum"), args.launches)
            print(f"{args.kernel} (1 PE, copy path): {ms * 1e3:.1f} us, {2 * n * 4 / ms / 1e6:.0f} GB/s")
        elif args.kernel in ("put_bw", "get_bw"):
            import ctypes as C
            from nvshmem_b200.bindings import host as H
            lib = C.CDLL(str(H.lib_path("libbshmem_devtest.so")))
            H.load().nvshmemx_b200_module_sync()
            size, iters = 256 << 20, 4
            sym = nv.tensor((size,), torch.uint8)
            local = torch.empty(size, dtype=torch.uint8, device=dev)
            counter = torch.zeros(1, dtype=torch.int32, device=dev)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            call = lambda: lib.perf_bw(C.c_void_p(sym.data_ptr()), C.c_void_p(local.data_ptr()), C.c_size_t(size), 0, iters, 2, int(args.kernel == "get_bw"), 32, 1024,
                                       C.c_void_p(counter.data_ptr()), stream)
            ms = timed(call, args.launches)
            print(f"{args.kernel} (block scope, 32 CTAs x 1024 threads, own heap): {ms * 1e3 / iters:.1f} us per {size >> 20} MB, {2 * size * iters / ms / 1e6:.0f} GB/s read+write")
        else:
            raise SystemExit(f"unknown kernel {args.kernel}")
    finally:
        nv.finalize()


if __name__ == "__main__":
    main()
