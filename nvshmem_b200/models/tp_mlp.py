"""Tensor-parallel transformer MLP: fused all-gather->GEMM, GELU, fused GEMM->reduce-scatter.

Input and output are token shards ``[tokens/npes, hidden]`` (sequence parallel).  With one PE it is
an ordinary MLP whose GEMMs run on the tcgen05 kernel.  ``reference`` computes the same block in
fp32 with plain torch for the numerics tests.
"""
from __future__ import annotations

import torch

from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _OpCache


class TensorParallelMLP(torch.nn.Module):
    def __init__(self, hidden: int, ffn: int, tokens: int, init_std: float = 0.02):
        super().__init__()
        self.cache = _OpCache()
        self.up = ColumnParallelLinear(hidden, ffn, tokens, self.cache, init_std)
        self.down = RowParallelLinear(ffn, hidden, tokens, self.cache, init_std)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        h = self.up(x_shard)
        h = torch.nn.functional.gelu(h, approximate="tanh")
        return self.down(h)

    @torch.no_grad()
    def reference(self, x_full: torch.Tensor, w_up_full: torch.Tensor | None = None, w_down_full: torch.Tensor | None = None) -> torch.Tensor:
        """fp32 result for the whole token range given full weights (defaults: this rank's, valid for one PE)."""
        w1 = (w_up_full if w_up_full is not None else self.up.weight).float()
        w2 = (w_down_full if w_down_full is not None else self.down.weight).float()
        h = torch.nn.functional.gelu((x_full.float() @ w1.t()).to(torch.bfloat16).float(), approximate="tanh").to(torch.bfloat16).float()
        return h @ w2.t()

    def close(self):
        self.cache.close()
