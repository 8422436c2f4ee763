"""Model blocks that run on the fused tensor-parallel and expert-parallel kernels."""
from .tp_mlp import TensorParallelMLP  # noqa: F401
from .moe_block import ExpertParallelMoE  # noqa: F401
