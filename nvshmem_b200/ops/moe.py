"""Expert-parallel MoE dispatch / combine on the fused NVLink kernels (``libbshmem_fused.so``).

``MoeDispatchCombine(T, H, K, E)`` owns the symmetric receive buffer, the expert-output buffer, the
count matrix and the flag block.  ``dispatch(x, topk_idx)`` returns the rows this rank's experts
received, grouped by local expert (``expert_offsets`` gives the group boundaries); after the expert
MLPs have written ``expert_out`` (same row numbering) ``combine(topk_idx, topk_weight)`` returns the
weighted sum for this rank's tokens.  ``payload="fp8"`` sends e4m3 with one fp32 scale per 128 values.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from .fused_gemm import fused_lib, _error_flag

MAX_PES, MAX_TOPK = 8, 16


class MoeError(RuntimeError):
    pass


class _DispatchArgs(C.Structure):
    _fields_ = [("T", C.c_int), ("H", C.c_int), ("K", C.c_int), ("E", C.c_int), ("rank", C.c_int), ("npes", C.c_int), ("payload", C.c_int), ("cap_rows", C.c_int),
                ("epoch", C.c_uint64), ("wait_limit_ms", C.c_uint32), ("max_ctas", C.c_int), ("error_flag", C.c_void_p), ("x", C.c_void_p), ("topk_idx", C.c_void_p),
                ("recv_x", C.c_void_p * MAX_PES), ("recv_scale", C.c_void_p * MAX_PES), ("slot_map", C.c_void_p), ("expert_offsets", C.c_void_p),
                ("src_offsets", C.c_void_p), ("counts", C.c_void_p * MAX_PES), ("flags", C.c_void_p * MAX_PES), ("scratch", C.c_void_p), ("dup_src", C.c_void_p * MAX_PES)]


class _CombineArgs(C.Structure):
    _fields_ = [("T", C.c_int), ("H", C.c_int), ("K", C.c_int), ("E", C.c_int), ("rank", C.c_int), ("npes", C.c_int), ("epoch", C.c_uint64),
                ("wait_limit_ms", C.c_uint32), ("max_ctas", C.c_int), ("error_flag", C.c_void_p), ("y", C.c_void_p * MAX_PES), ("topk_idx", C.c_void_p),
                ("topk_weight", C.c_void_p), ("slot_map", C.c_void_p), ("out", C.c_void_p), ("flags", C.c_void_p * MAX_PES), ("scratch", C.c_void_p)]


def _lib():
    lib = fused_lib()
    if not hasattr(lib, "_moe_ready"):
        lib.bshmem_moe_dispatch.restype = C.c_int
        lib.bshmem_moe_dispatch.argtypes = [C.POINTER(_DispatchArgs), C.c_void_p]
        lib.bshmem_moe_combine.restype = C.c_int
        lib.bshmem_moe_combine.argtypes = [C.POINTER(_CombineArgs), C.c_void_p]
        lib.bshmem_moe_scratch_bytes.restype = C.c_size_t
        lib.bshmem_moe_scratch_bytes.argtypes = [C.c_int]
        lib._moe_ready = True
    return lib


class MoeDispatchCombine:
    """Expert-parallel dispatch and combine.  ``dedup=True`` (with more than one PE): a token that goes to several
    experts of one PE crosses NVLink once and is replicated into its other rows by the receiving PE (with top-8 of 256
    experts on 8 PEs a token reaches 5.25 distinct PEs on average, so about a third of the link bytes go away).  The
    default is the per-pair form; ``BSHMEM_MOE_DEDUP=1`` turns the other one on for objects that do not say."""

    def __init__(self, T: int, H: int, K: int, E: int, payload: str = "bf16", cap_rows: int | None = None, wait_limit_ms: int = 0, dedup: bool | None = None):
        from .. import core
        self.core = core
        self.rank, self.npes = core.my_pe(), core.n_pes()
        if self.npes > MAX_PES or K > MAX_TOPK or E % self.npes or H % 128:
            raise MoeError("unsupported shape: npes <= 8, K <= 16, E divisible by npes, H divisible by 128")
        self.T, self.H, self.K, self.E, self.EL = T, H, K, E, E // self.npes
        self.fp8 = payload == "fp8"
        self.wait_limit_ms = wait_limit_ms
        # Worst case every pair of every rank lands on one PE; callers with balanced routing pass less.
        self.cap_rows = cap_rows or T * K * self.npes
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.epoch = 0
        row_bytes = H if self.fp8 else 2 * H
        sym = self.npes > 1
        alloc = (lambda shape, dt, zero=False: core.tensor(shape, dt, zero=zero)) if sym else (lambda shape, dt, zero=False: torch.zeros(shape, dtype=dt, device=self.device))
        self._sym = sym
        self.recv_raw = alloc((self.cap_rows, row_bytes), torch.uint8)
        self.recv_scale = alloc((self.cap_rows, H // 128), torch.float32) if self.fp8 else None
        self.expert_out = alloc((self.cap_rows, H), torch.bfloat16)
        if dedup is None:
            dedup = os.environ.get("BSHMEM_MOE_DEDUP", "0") == "1"
        self.dedup = bool(dedup) and sym
        self.dup_src = alloc((self.cap_rows,), torch.int32) if self.dedup else None
        self.counts = alloc((self.npes * E,), torch.int32, True)
        self.flags = alloc((4 * self.npes,), torch.int64, True)
        self.scratch = torch.zeros(_lib().bshmem_moe_scratch_bytes(E) // 4 + 64, dtype=torch.int32, device=self.device)
        self.slot_map = torch.empty(T, K, dtype=torch.int32, device=self.device)
        self.expert_offsets = torch.zeros(self.EL + 1, dtype=torch.int32, device=self.device)
        self.src_offsets = torch.zeros(self.EL, self.npes, dtype=torch.int32, device=self.device)
        self.out = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
        self._tensors = [t for t in (self.recv_raw, self.recv_scale, self.expert_out, self.counts, self.flags, self.dup_src) if t is not None]
        ptr = (lambda t, q: core.peer_ptr(t, q)) if sym else (lambda t, q: t.data_ptr())
        self._peers = {q: {"recv": ptr(self.recv_raw, q), "scale": ptr(self.recv_scale, q) if self.fp8 else 0, "y": ptr(self.expert_out, q),
                           "counts": ptr(self.counts, q), "flags": ptr(self.flags, q), "dup": ptr(self.dup_src, q) if self.dedup else 0} for q in range(self.npes)}
        if sym:
            core.barrier_all()
            torch.cuda.synchronize()

    @property
    def recv_x(self) -> torch.Tensor:
        """Received rows: ``[cap_rows, H]`` bf16, or e4m3 bytes viewed as ``torch.float8_e4m3fn``."""
        return self.recv_raw.view(torch.float8_e4m3fn) if self.fp8 else self.recv_raw.view(torch.bfloat16)

    def dequantized(self, rows: int) -> torch.Tensor:
        """fp8 payload back to fp32 (tests and reference expert MLPs)."""
        q = self.recv_raw[:rows].view(torch.float8_e4m3fn).float().view(rows, self.H // 128, 128)
        return (q * self.recv_scale[:rows].unsqueeze(-1)).view(rows, self.H)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor):
        if x.shape != (self.T, self.H) or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise MoeError("x must be contiguous bf16 [T, H]")
        if topk_idx.shape != (self.T, self.K) or topk_idx.dtype != torch.int32 or not topk_idx.is_contiguous():
            raise MoeError("topk_idx must be contiguous int32 [T, K]")
        self.epoch += 1
        a = _DispatchArgs()
        a.T, a.H, a.K, a.E, a.rank, a.npes = self.T, self.H, self.K, self.E, self.rank, self.npes
        a.payload, a.cap_rows, a.epoch, a.wait_limit_ms = int(self.fp8), self.cap_rows, self.epoch, self.wait_limit_ms
        a.error_flag = _error_flag(self.device).data_ptr()
        a.x, a.topk_idx = x.data_ptr(), topk_idx.data_ptr()
        for q in range(self.npes):
            a.recv_x[q], a.recv_scale[q] = self._peers[q]["recv"], self._peers[q]["scale"]
            a.counts[q], a.flags[q] = self._peers[q]["counts"], self._peers[q]["flags"]
            a.dup_src[q] = self._peers[q]["dup"]
        a.slot_map, a.expert_offsets, a.src_offsets = self.slot_map.data_ptr(), self.expert_offsets.data_ptr(), self.src_offsets.data_ptr()
        a.scratch = self.scratch.data_ptr()
        st = _lib().bshmem_moe_dispatch(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise MoeError(f"bshmem_moe_dispatch failed with status {st}")
        return self.recv_x, self.expert_offsets

    def combine(self, topk_idx: torch.Tensor, topk_weight: torch.Tensor) -> torch.Tensor:
        if topk_weight.shape != (self.T, self.K) or topk_weight.dtype != torch.float32 or not topk_weight.is_contiguous():
            raise MoeError("topk_weight must be contiguous fp32 [T, K]")
        a = _CombineArgs()
        a.T, a.H, a.K, a.E, a.rank, a.npes = self.T, self.H, self.K, self.E, self.rank, self.npes
        a.epoch, a.wait_limit_ms = self.epoch, self.wait_limit_ms
        a.error_flag = _error_flag(self.device).data_ptr()
        for q in range(self.npes):
            a.y[q], a.flags[q] = self._peers[q]["y"], self._peers[q]["flags"]
        a.topk_idx, a.topk_weight, a.slot_map, a.out = topk_idx.data_ptr(), topk_weight.data_ptr(), self.slot_map.data_ptr(), self.out.data_ptr()
        a.scratch = self.scratch.data_ptr()
        st = _lib().bshmem_moe_combine(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise MoeError(f"bshmem_moe_combine failed with status {st}")
        return self.out

    def close(self) -> None:
        if self._sym:
            torch.cuda.synchronize()
            for t in self._tensors:
                self.core.free_tensor(t)
        self._tensors = []
