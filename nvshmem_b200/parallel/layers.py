"""Sequence-parallel tensor-parallel linear layers whose collectives are fused into the GEMM kernel.

Activations are sharded by rows (tokens) between layers, Megatron sequence-parallel style:

* :class:`ColumnParallelLinear`  – input ``[M/npes, K]`` shard, weight ``[N/npes, K]``; forward is the fused
  all-gather -> GEMM and yields ``[M, N/npes]``.
* :class:`RowParallelLinear`     – input ``[M, K/npes]``, weight ``[N, K/npes]``; forward is the fused
  GEMM -> reduce-scatter and yields the ``[M/npes, N]`` shard.

The backward passes reuse the same fused kernels with the roles swapped (the gradient of an
all-gather is a reduce-scatter and vice versa); weight gradients use the plain tcgen05 GEMM.
Every fused result is written by the kernel straight into a tensor of its own (``out=``): no
result is copied out of an operator-owned buffer.
"""
from __future__ import annotations

import torch

from ..ops import fused_gemm as fg


class _OpCache:
    """Fused-op objects own symmetric buffers, so they are created once per shape and reused."""

    def __init__(self):
        self.rs: dict = {}
        self.ag: dict = {}

    def reduce_scatter(self, M: int, N: int) -> fg.GemmReduceScatter:
        key = (M, N)
        if key not in self.rs:
            self.rs[key] = fg.GemmReduceScatter(M, N, mode="rs")
        return self.rs[key]

    def all_gather(self, M: int, K: int, owner=None) -> fg.AllGatherGemm:
        """`owner` keeps a private gathered buffer (a layer's forward input must survive until its
        backward); without it the buffer is shared by every user of the shape (transient use)."""
        key = (M, K, id(owner) if owner is not None else None)
        if key not in self.ag:
            self.ag[key] = fg.AllGatherGemm(M, K)
        return self.ag[key]

    def close(self):
        for op in list(self.rs.values()) + list(self.ag.values()):
            op.close()
        self.rs.clear()
        self.ag.clear()


def _t(x: torch.Tensor) -> torch.Tensor:
    return x.t().contiguous()


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, cache: _OpCache, M: int, owner):
        K = x_shard.shape[1]
        ag = cache.all_gather(M, K, owner)
        if x_shard.data_ptr() != ag.shard.data_ptr():  # a producer may have written the shard in place
            ag.shard.copy_(x_shard)
        y = ag(weight, out=torch.empty(M, weight.shape[0], dtype=torch.bfloat16, device=weight.device))
        ctx.save_for_backward(weight)
        ctx.cache, ctx.M, ctx.K = cache, M, K
        ctx.x_full = ag.gathered  # valid until the next forward of the same shape
        return y

    @staticmethod
    def backward(ctx, dy):
        (weight,) = ctx.saved_tensors
        dy = dy.contiguous()
        x_full = ctx.x_full
        # dW[Nl, K] = dY^T @ X_full
        dw = fg.gemm(_t(dy), _t(x_full))
        # dX_shard[M/n, K] = reduce_scatter(dY[M, Nl] @ W[Nl, K])
        rs = ctx.cache.reduce_scatter(ctx.M, ctx.K)
        dx = rs(dy, _t(weight), out=torch.empty(rs.rows, ctx.K, dtype=torch.bfloat16, device=dy.device))
        return dx, dw, None, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cache: _OpCache):
        M, N = x.shape[0], weight.shape[0]
        rs = cache.reduce_scatter(M, N)
        y = rs(x.contiguous(), weight, out=torch.empty(rs.rows, N, dtype=torch.bfloat16, device=x.device))
        ctx.save_for_backward(x, weight)
        ctx.cache, ctx.M, ctx.N = cache, M, N
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        # dX[M, Kl] = all_gather(dY_shard)[M, N] @ W[N, Kl]
        ag = ctx.cache.all_gather(ctx.M, ctx.N)
        ag.shard.copy_(dy_shard)
        wt = _t(weight)
        dx = ag(wt, out=torch.empty(ctx.M, wt.shape[0], dtype=torch.bfloat16, device=dy_shard.device))
        # dW[N, Kl] = dY_full^T @ X
        dw = fg.gemm(_t(ag.gathered), _t(x))
        return dx, dw, None


class ColumnParallelLinear(torch.nn.Module):
    """``y[M, out/npes] = all_gather(x_shard)[M, in] @ W_shard[out/npes, in]^T`` with the gather fused into the GEMM."""

    def __init__(self, in_features: int, out_features: int, tokens: int, cache: _OpCache | None = None, init_std: float = 0.02, device=None):
        super().__init__()
        from .. import core
        self.npes, self.rank = core.n_pes(), core.my_pe()
        assert out_features % self.npes == 0 and tokens % self.npes == 0
        self.tokens = tokens
        self.cache = cache or _OpCache()
        device = device or torch.device("cuda", torch.cuda.current_device())
        w = torch.empty(out_features // self.npes, in_features, device=device, dtype=torch.float32).normal_(0.0, init_std)
        self.weight = torch.nn.Parameter(w.to(torch.bfloat16))

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _ColumnParallelFn.apply(x_shard, self.weight, self.cache, self.tokens, self)


class RowParallelLinear(torch.nn.Module):
    """``y_shard[M/npes, out] = reduce_scatter(x[M, in/npes] @ W_shard[out, in/npes]^T)`` with the reduction fused into the epilogue."""

    def __init__(self, in_features: int, out_features: int, tokens: int, cache: _OpCache | None = None, init_std: float = 0.02, device=None):
        super().__init__()
        from .. import core
        self.npes, self.rank = core.n_pes(), core.my_pe()
        assert in_features % self.npes == 0 and tokens % self.npes == 0
        self.tokens = tokens
        self.cache = cache or _OpCache()
        device = device or torch.device("cuda", torch.cuda.current_device())
        w = torch.empty(out_features, in_features // self.npes, device=device, dtype=torch.float32).normal_(0.0, init_std)
        self.weight = torch.nn.Parameter(w.to(torch.bfloat16))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _RowParallelFn.apply(x, self.weight, self.cache)
