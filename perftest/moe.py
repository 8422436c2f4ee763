"""Expert-parallel dispatch / combine against an NCCL all-to-all baseline.

Default: 4096 tokens per rank, hidden 7168, 256 experts, top-8 from the softmax of N(0,1) logits; bf16 and fp8
(e4m3 + 1x128 fp32 scales) dispatch, bf16 weighted combine.  Reports microseconds per layer and GB/s of payload
that a pair-by-pair exchange moves over NVLink (rows whose expert lives on another rank), and the fraction of
770 GB/s.  Dispatch runs twice: sending a token once per destination rank (the default; `sent_GB` is what then
crosses the links) and once per (token, expert) pair.
The baseline does what a framework without fused kernels does: sort pairs by destination, exchange counts,
all_to_all_single the rows, and for combine the reverse plus an index_add of the weighted rows.

  torchrun --nproc-per-node 8 -m perftest.moe
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from .common import Env


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    env = Env()
    n, me = env.world, env.rank
    from nvshmem_b200.ops.moe import MoeDispatchCombine
    from nvshmem_b200.ops import fused_gemm as fg
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    EL = E // n
    g = torch.Generator(device=env.dev).manual_seed(42 + me)
    x = torch.randn(T, H, device=env.dev, generator=g).to(torch.bfloat16)
    probs = torch.randn(T, E, device=env.dev, generator=g).softmax(-1)
    w, idx = probs.topk(K, dim=-1)
    idx = idx.to(torch.int32).contiguous()
    w = w.float().contiguous()
    remote_pairs = int(((idx // EL) != me).sum())
    dest = (idx // EL).long()
    reached = torch.zeros(T, n, dtype=torch.bool, device=env.dev).scatter_(1, dest, True)
    reached[:, me] = False
    remote_once = int(reached.sum())  # (token, remote rank) pairs: what crosses NVLink when a token is sent once per rank
    cap = int(T * K * 2.0) if n > 1 else T * K  # balanced routing: twice the mean is ample
    for payload, row_bytes, dedup in (("bf16", 2 * H, True), ("bf16", 2 * H, False), ("fp8", H + H // 128 * 4, True), ("fp8", H + H // 128 * 4, False)):
        if n == 1 and not dedup:
            continue
        moe = MoeDispatchCombine(T, H, K, E, payload=payload, cap_rows=cap, dedup=dedup)
        ms = env.time_ms(lambda: moe.dispatch(x, idx), iters=args.iters, warmup=3)
        fg.check_errors()
        gb = remote_pairs * row_bytes / 1e9
        sent = (remote_once if moe.dedup else remote_pairs) * row_bytes / 1e9
        env.record(test=f"moe_dispatch_{payload}" + ("" if dedup else "_per_pair"), us=round(ms * 1e3, 1), nvlink_GB=round(gb, 4), GBps=round(gb / (ms * 1e-3), 1),
                   fraction_of_770=round(gb / (ms * 1e-3) / 770, 3), sent_GB=round(sent, 4), sent_GBps=round(sent / (ms * 1e-3), 1), npes=n, tokens=T, hidden=H, experts=E, topk=K)
        if payload == "bf16" and dedup:
            rows = int(moe.expert_offsets[-1])
            moe.expert_out[:rows] = moe.recv_x[:rows]
            ms = env.time_ms(lambda: moe.combine(idx, w), iters=args.iters, warmup=3)
            fg.check_errors()
            gb = remote_pairs * 2 * H / 1e9
            env.record(test="moe_combine_bf16", us=round(ms * 1e3, 1), nvlink_GB=round(gb, 4), GBps=round(gb / (ms * 1e-3), 1), fraction_of_770=round(gb / (ms * 1e-3) / 770, 3), npes=n)
        moe.close()
    if n > 1:
        # ---- NCCL baseline
        flat_e = idx.flatten().long()
        def nccl_dispatch():
            order = torch.argsort(flat_e, stable=True)
            rows = x[order // K]
            send_counts = torch.bincount(flat_e // EL, minlength=n)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            sc, rc = send_counts.tolist(), recv_counts.tolist()
            recv = torch.empty(sum(rc), H, dtype=torch.bfloat16, device=env.dev)
            dist.all_to_all_single(recv, rows, rc, sc)
            return recv, order, sc, rc
        ms = env.time_ms(lambda: nccl_dispatch(), iters=args.iters, warmup=3)
        gb = remote_pairs * 2 * H / 1e9
        env.record(test="moe_dispatch_bf16_nccl", us=round(ms * 1e3, 1), GBps=round(gb / (ms * 1e-3), 1), npes=n)
        recv, order, sc, rc = nccl_dispatch()
        def nccl_combine():
            back = torch.empty(T * K, H, dtype=torch.bfloat16, device=env.dev)
            dist.all_to_all_single(back, recv, sc, rc)
            out = torch.zeros(T, H, dtype=torch.float32, device=env.dev)
            out.index_add_(0, order // K, back.float() * w.flatten()[order].unsqueeze(1))
            return out.to(torch.bfloat16)
        ms = env.time_ms(lambda: nccl_combine(), iters=args.iters, warmup=3)
        env.record(test="moe_combine_bf16_nccl", us=round(ms * 1e3, 1), GBps=round(gb / (ms * 1e-3), 1), npes=n)
    env.finish()


if __name__ == "__main__":
    main()
