"""Expert-parallel mixture-of-experts block on the fused dispatch / combine kernels.

Each rank holds ``E / npes`` experts (a gated MLP each).  ``forward(x)``:
router logits -> softmax -> top-k -> ``MoeDispatchCombine.dispatch`` (tokens travel to the ranks of
their experts, grouped by expert) -> the local experts' MLPs over their row groups -> ``combine``
(the weighted sum comes back to the token's rank).  The experts run as two grouped GEMMs on the
tcgen05 kernel (``ops.fused_gemm.grouped_gemm``): the group boundaries stay on the device, the gated
activation is applied in the first GEMM's epilogue, and the second GEMM writes straight into the
buffer that ``combine`` reads; nothing is synchronised with the host between dispatch and combine.
Inference path: no autograd through the exchange.
(the reference's counterpart is the data movement of examples/moe_shuffle.cu; the experts and the
router are this framework's)
"""
from __future__ import annotations

import torch

from ..ops import fused_gemm as fg
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
        # The grouped tcgen05 GEMM needs 256-column output tiles and 64-deep K steps; other shapes use torch matmuls.
        self.grouped = (2 * ffn) % 256 == 0 and hidden % 256 == 0 and ffn % 64 == 0 and self.EL <= fg.MAX_GROUPS and not self.fp8_payload(payload)
        if self.grouped:
            self.w_in_gated = fg.interleave_gate_up(self.w_in.data)   # rows reordered for the fused gated activation
            self.act_buf = torch.empty(self.exchange.cap_rows, ffn, dtype=torch.bfloat16, device=dev)

    @staticmethod
    def fp8_payload(payload: str) -> bool:
        return payload == "fp8"

    def route(self, x: torch.Tensor):
        if self.T % 128 == 0 and self.E % 256 == 0 and self.H % 64 == 0:
            logits = fg.gemm(x, self.router).float()   # the router is a GEMM like any other
        else:
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
        if self.grouped:
            # two grouped GEMMs over the expert segments; `offsets` never leaves the device
            fg.grouped_gemm(recv, self.w_in_gated, offsets, out=self.act_buf, act="swiglu")
            fg.grouped_gemm(self.act_buf, self.w_out, offsets, out=self.exchange.expert_out)
        else:
            offs = offsets.tolist()  # group boundaries on the host to slice per-expert matmuls
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
