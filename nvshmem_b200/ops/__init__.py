"""Torch-facing operators built on the fused sm_100a kernels."""
from .fused_gemm import (FusedGemmError, gemm, GemmReduceScatter, AllGatherGemm, fused_lib)  # noqa: F401
from .moe import MoeDispatchCombine, MoeError  # noqa: F401
