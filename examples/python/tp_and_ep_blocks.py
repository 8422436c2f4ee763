"""The fused products from Python: a tensor-parallel MLP (all-gather -> GEMM, GEMM -> reduce-scatter in one
kernel each) and an expert-parallel MoE block (dispatch / combine kernels).

  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/python/tp_and_ep_blocks.py

(the reference shows these patterns as examples/gemm_allreduce and examples/moe_shuffle.cu)
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem_b200.core as nv  # noqa: E402
from nvshmem_b200.models import ExpertParallelMoE, TensorParallelMLP  # noqa: E402
from nvshmem_b200.ops import fused_gemm as fg  # noqa: E402


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.init(device=local_rank, initializer_method="torch")
    me, n = nv.my_pe(), nv.n_pes()
    torch.manual_seed(1 + me)

    tokens, hidden, ffn = 1024 * n, 4096, 2048 * n
    mlp = TensorParallelMLP(hidden, ffn, tokens)
    x_shard = torch.randn(tokens // n, hidden, device="cuda").to(torch.bfloat16)   # sequence-parallel input: my rows
    with torch.no_grad():
        ms = timed(lambda: mlp(x_shard))
    fg.check_errors()
    if me == 0:
        print(f"TP MLP {tokens} x {hidden} x {ffn} on {n} PEs: {ms:.3f} ms per forward")

    t_local, experts, topk = 2048, 8 * n, 4
    moe = ExpertParallelMoE(t_local, hidden, 1024, experts, topk)
    xt = torch.randn(t_local, hidden, device="cuda").to(torch.bfloat16)
    ms = timed(lambda: moe(xt), iters=5)
    fg.check_errors()
    if me == 0:
        print(f"EP MoE block {t_local} tokens/rank, {experts} experts, top-{topk}: {ms:.3f} ms per forward")
    moe.close()
    mlp.close()
    nv.finalize()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
