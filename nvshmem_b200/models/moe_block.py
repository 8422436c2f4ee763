"""Expert-parallel mixture-of-experts block on the fused dispatch / combine kernels.

Each rank holds ``E / npes`` experts (a gated MLP each).  ``forward(x)``:
router logits -> softmax -> top-k -> ``MoeDispatchCombine.dispatch`` (tokens travel to the ranks of
their experts, grouped by expert) -> the local experts' MLPs over their row groups -> ``combine``
(the weighted sum comes back to the token's rank).  Inference path: no autograd through the exchange.
(the reference's counterpart is the data movement of examples/moe_shuffle.cu; the experts and the
router are this framework's)
"""
from __future__ import annotations

import torch

from ..ops.moe import MoeDispatchCombine


class ExpertParallelMoE(torch.nn.Module):
    def __init__(self, tokens: int, hidden: int, ffn: int, experts: int, topk: int, payload: str = "bf16", seed: int = 0, wait_limit_ms: int = 0):
        super().__init__()
        from .. import core
        self.rank, self.npes = core.my_pe(), core.n_pes()
        self.T, self.H, self.F, self.E, self.K = tokens, hidden, ffn, experts, topk
        self.EL = experts // self.npes
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device="cpu").manual_seed(seed)  # the same router and experts on every rank, sliced by ownership
        router = torch.randn(experts, hidden, generator=g) * hidden ** -0.5
        w_in = torch.randn(experts, 2 * ffn, hidden, generator=g) * 0.02
        w_out = torch.randn(experts, hidden, ffn, generator=g) * 0.02
        mine = slice(self.rank * self.EL, (self.rank + 1) * self.EL)
        self.router = torch.nn.Parameter(router.to(dev, torch.bfloat16), requires_grad=False)
        self.w_in = torch.nn.Parameter(w_in[mine].to(dev, torch.bfloat16).contiguous(), requires_grad=False)    # [EL, 2F, H]: gate and up projections
        self.w_out = torch.nn.Parameter(w_out[mine].to(dev, torch.bfloat16).contiguous(), requires_grad=False)  # [EL, H, F]
        self.exchange = MoeDispatchCombine(tokens, hidden, topk, experts, payload=payload, wait_limit_ms=wait_limit_ms)

    def route(self, x: torch.Tensor):
        logits = (x @ self.router.t()).float()
        weight, idx = logits.softmax(-1).topk(self.K, dim=-1)
        weight = weight / weight.sum(-1, keepdim=True)
        return idx.to(torch.int32).contiguous(), weight.contiguous()

    def experts_forward(self, rows: torch.Tensor, offsets: list[int]) -> None:
        """Runs local expert e over rows [offsets[e], offsets[e+1]) and writes the exchange's expert_out."""
        out = self.exchange.expert_out
        for e in range(self.EL):
            lo, hi = offsets[e], offsets[e + 1]
            if hi == lo:
                continue
            h = rows[lo:hi] @ self.w_in[e].t()
            gate, up = h[:, :self.F], h[:, self.F:]
            out[lo:hi] = (torch.nn.functional.silu(gate.float()).to(torch.bfloat16) * up) @ self.w_out[e].t()

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        idx, weight = self.route(x)
        recv, offsets = self.exchange.dispatch(x, idx)
        offs = offsets.tolist()  # group boundaries are needed on the host to slice the grouped GEMMs
        rows = self.exchange.dequantized(offs[-1]).to(torch.bfloat16) if self.exchange.fp8 else recv
        self.experts_forward(rows, offs)
        return self.exchange.combine(idx, weight)

    def close(self) -> None:
        self.exchange.close()


@torch.no_grad()
def reference_forward(x: torch.Tensor, router: torch.Tensor, w_in: torch.Tensor, w_out: torch.Tensor, topk: int) -> torch.Tensor:
    """Plain PyTorch fp32 version of the block with all experts on one device (test oracle).
    w_in: [E, 2F, H], w_out: [E, H, F]."""
    F = w_out.shape[2]
    logits = (x @ router.t()).float()
    weight, idx = logits.softmax(-1).topk(topk, dim=-1)
    weight = weight / weight.sum(-1, keepdim=True)
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(w_in.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ w_in[e].float().t()
        y = (torch.nn.functional.silu(h[:, :F]) * h[:, F:]) @ w_out[e].float().t()
        out.index_add_(0, tok, y * weight[tok, slot].unsqueeze(-1))
    return out
