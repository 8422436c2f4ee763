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


class TensorParallelMLPStack:
    """``layers`` tensor-parallel MLP blocks applied one after the other to a token shard, forward only
    (what a serving step of the MLP part of a transformer does).

    Per block: fused all-gather -> GEMM with the tanh-GELU applied in the GEMM's epilogue, then fused
    GEMM -> reduce-scatter whose result is written straight into this rank's shard of the all-gather
    buffer, where the next block picks it up: two kernels and one team sync per block, and no copy
    between blocks.  The blocks share one all-gather buffer and one set of reduce-scatter buffers.

    ``input_shard`` is where the caller puts this rank's ``[tokens/npes, hidden]`` tokens (it may be the
    target of a host-to-device copy); ``forward()`` returns this rank's ``[tokens/npes, hidden]`` result in a
    tensor owned by the object.

    ``gather="fused"`` (default) is the above.  ``gather="collective"`` runs the all-gather as the library's
    on-stream ``fcollect`` (its own kernel) followed by the plain GEMM with the same fused GELU: three kernels per
    block, for comparison and as the path to fall back to when the fused all-gather cannot be used.
    """

    def __init__(self, hidden: int, ffn: int, tokens: int, layers: int, init_std: float = 0.02, seed: int | None = None, gather: str = "fused",
                 wait_limit_ms: int = 0):
        from .. import core
        from ..ops import fused_gemm as fg
        self.npes, self.rank = core.n_pes(), core.my_pe()
        assert ffn % self.npes == 0 and tokens % self.npes == 0
        self.hidden, self.ffn, self.tokens, self.layers = hidden, ffn, tokens, layers
        dev = torch.device("cuda", torch.cuda.current_device())
        gen = torch.Generator(device=dev)
        if seed is not None:
            gen.manual_seed(seed)
        fl = ffn // self.npes
        self.w_up = [torch.empty(fl, hidden, device=dev, dtype=torch.float32).normal_(0.0, init_std, generator=gen).to(torch.bfloat16) for _ in range(layers)]
        self.w_down = [torch.empty(hidden, fl, device=dev, dtype=torch.float32).normal_(0.0, init_std, generator=gen).to(torch.bfloat16) for _ in range(layers)]
        if gather not in ("fused", "collective"):
            raise ValueError("gather is 'fused' or 'collective'")
        self.gather = gather if self.npes > 1 else "fused"
        self._core, self._fg = core, fg
        if self.gather == "fused":
            self.ag = fg.AllGatherGemm(tokens, hidden, wait_limit_ms=wait_limit_ms)
            self._shard = self.ag.shard
        else:
            self.ag = None
            self.gathered = core.tensor((tokens, hidden), torch.bfloat16)
            self._shard = core.tensor((tokens // self.npes, hidden), torch.bfloat16)
        self.rs = fg.GemmReduceScatter(tokens, hidden, mode="rs", wait_limit_ms=wait_limit_ms)
        self.h = torch.empty(tokens, fl, dtype=torch.bfloat16, device=dev)
        self.out = torch.empty(tokens // self.npes, hidden, dtype=torch.bfloat16, device=dev)
        # GEMM, GEMM (+ the team sync before each fused all-gather, or the fcollect kernel)
        self.kernels_per_forward = layers * (3 if self.npes > 1 else 2)

    @property
    def input_shard(self) -> torch.Tensor:
        return self._shard

    @torch.no_grad()
    def forward(self) -> torch.Tensor:
        for l in range(self.layers):
            if self.gather == "fused":
                self.ag(self.w_up[l], out=self.h, act="gelu_tanh")
            else:
                # fcollect ends with a team barrier, so the previous block's readers of `gathered` are done before it is rewritten
                self._core.fcollect(self._core.Teams.TEAM_WORLD, self.gathered, self._shard, stream=torch.cuda.current_stream())
                self._fg.gemm(self.gathered, self.w_up[l], out=self.h, act="gelu_tanh")
            self.rs(self.h, self.w_down[l], out=self._shard if l + 1 < self.layers else self.out)
        return self.out

    __call__ = forward

    @torch.no_grad()
    def reference(self, x_full: torch.Tensor, w_up_full: list, w_down_full: list) -> torch.Tensor:
        """The same stack in fp32 with plain torch on full weights, rounding to bf16 where the kernels do."""
        x = x_full.float()
        for w1, w2 in zip(w_up_full, w_down_full):
            h = torch.nn.functional.gelu(x @ w1.float().t(), approximate="tanh").to(torch.bfloat16).float()
            x = (h @ w2.float().t()).to(torch.bfloat16).float()
        return x

    def close(self):
        if self.ag is not None:
            self.ag.close()
        else:
            torch.cuda.synchronize()
            self._core.free_tensor(self.gathered)
            self._core.free_tensor(self._shard)
        self.rs.close()
