"""Tensor- and expert-parallel building blocks on the fused kernels."""
from .layers import ColumnParallelLinear, RowParallelLinear  # noqa: F401
