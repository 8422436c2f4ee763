"""Tensor-parallel GEMMs fused with their collective (``libbshmem_fused.so``).

* :func:`gemm` – plain ``x @ w.T`` on the tcgen05 kernel (what one GPU runs).
* :class:`GemmReduceScatter` – row-parallel linear: every rank multiplies its K-slice; with an NVLink
  multicast window the partial tiles stay in the producing GPU's staging buffer and the owner of a
  tile reads their sum through the switch (``multimem.ld_reduce``) inside the same kernel, otherwise
  the epilogue pushes partial tiles into the owning rank's receive slots and reduces there
  (``mode="rs"``); ``mode="ar"`` additionally delivers the reduced tile to all ranks.
* :class:`AllGatherGemm` – column-parallel linear: two spare warps of every CTA (or, as an option, copy engines)
  spread the local activation shard to all peers while the GEMM consumes shards as they land.

Weights use torch's Linear layout ``[out_features, in_features]``; activations are ``[tokens,
in_features]``; everything is bf16 with fp32 accumulation.  The collective variants keep their
buffers in the symmetric heap; a call counter (epoch) replaces flag resets.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..bindings import host as H

MAX_PES = 8
MODES = {"plain": 0, "rs": 1, "ar": 2, "ag": 3, "grouped": 4}
ACTS = {None: 0, "none": 0, "gelu_tanh": 1, "swiglu": 2}
MAX_GROUPS = 256
_lib = None


class FusedGemmError(RuntimeError):
    pass


class _Args(C.Structure):
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("out", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("rank", C.c_int), ("npes", C.c_int),
                ("mode", C.c_int), ("epoch", C.c_uint64), ("wait_limit_ms", C.c_uint32), ("max_ctas", C.c_int), ("n_comm", C.c_int), ("error_flag", C.c_void_p),
                ("recv_local", C.c_void_p), ("recv_peer", C.c_void_p * MAX_PES), ("flags_local", C.c_void_p), ("flags_peer", C.c_void_p * MAX_PES),
                ("out_peer", C.c_void_p * MAX_PES), ("ag_peer", C.c_void_p * MAX_PES), ("ag_flags_local", C.c_void_p), ("ag_flags_peer", C.c_void_p * MAX_PES), ("out_mc", C.c_void_p),
                ("stage_local", C.c_void_p), ("stage_mc", C.c_void_p), ("act", C.c_int), ("ag_external", C.c_int), ("group_offsets", C.c_void_p), ("groups", C.c_int)]


_ERRORS = {1: "bad arguments", 2: "shape: M must be a multiple of 128*npes, N of 256, K of 64", 3: "operands must be 16-byte aligned", 4: "CUDA driver/runtime error"}


def fused_lib() -> C.CDLL:
    """Loads the fused-kernel library; a missing library is an error (no fallback path exists)."""
    global _lib
    if _lib is None:
        path = H.lib_path("libbshmem_fused.so")
        if not path.exists():
            raise ImportError(f"{path} is missing: build it with `python -m nvshmem_b200.utils.build`")
        _lib = C.CDLL(str(path))
        _lib.bshmem_fused_gemm.restype = C.c_int
        _lib.bshmem_fused_gemm.argtypes = [C.POINTER(_Args), C.c_void_p]
    return _lib


_err_flags: dict[int, torch.Tensor] = {}


def _error_flag(device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _err_flags:
        _err_flags[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_flags[idx]


def check_errors(device=None) -> None:
    """Raises if a fused kernel gave up on a wait since the last check (synchronises the device)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    flag = _error_flag(device)
    v = int(flag.item())
    if v:
        flag.zero_()
        raise FusedGemmError(f"a fused kernel abandoned a bounded wait (code {v}): a peer did not deliver its tiles in time")


def take_error(device=None) -> int:
    """Returns the error word of the fused kernels on `device` and clears it (0: no kernel gave up on a wait since the
    last check).  Synchronises the device.  For callers that want to react instead of raising."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    flag = _error_flag(device)
    v = int(flag.item())
    if v:
        flag.zero_()
    return v


def _launch(args: _Args, stream) -> None:
    st = fused_lib().bshmem_fused_gemm(C.byref(args), C.c_void_p(stream))
    if st != 0:
        raise FusedGemmError(f"bshmem_fused_gemm: {_ERRORS.get(st, st)}")


def _check_operands(x: torch.Tensor, w: torch.Tensor) -> None:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise FusedGemmError("operands must be bfloat16")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise FusedGemmError(f"shape mismatch: x {tuple(x.shape)} w {tuple(w.shape)}")
    if not x.is_contiguous() or not w.is_contiguous():
        raise FusedGemmError("operands must be contiguous")


def _check_out(out: torch.Tensor, rows: int, cols: int) -> None:
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (rows, cols) or not out.is_contiguous() or out.data_ptr() % 16:
        raise FusedGemmError(f"`out` must be a contiguous, 16-byte aligned bfloat16 tensor of shape {(rows, cols)}")


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, max_ctas: int = 0, act: str | None = None) -> torch.Tensor:
    """``act(x[M,K] @ w[N,K].T)`` -> bf16 ``[M,N]`` on the tcgen05/TMEM kernel; ``act`` is None or ``"gelu_tanh"``
    (applied to the fp32 accumulators in the epilogue)."""
    _check_operands(x, w)
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    else:
        _check_out(out, M, N)
    a = _Args()
    a.act = ACTS[act]
    a.A, a.B, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.M, a.N, a.K, a.rank, a.npes, a.mode = M, N, K, 0, 1, MODES["plain"]
    a.epoch, a.max_ctas = 1, max_ctas
    a.error_flag = _error_flag(x.device).data_ptr()
    _launch(a, torch.cuda.current_stream().cuda_stream)
    return out


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, out: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
    """Grouped GEMM on the tcgen05 kernel: the rows of ``x[R, K]`` fall into ``G`` consecutive groups with boundaries
    ``group_offsets`` (int32 ``[G + 1]`` ON THE DEVICE: the kernel reads them, nothing is synchronised with the
    host), ``w`` is ``[G, N, K]``, and rows of group ``g`` are multiplied by ``w[g].T``.  Rows at or beyond
    ``group_offsets[G]`` are not written.  This is the contraction of a mixture-of-experts layer after dispatch.

    ``act="swiglu"``: each 64 rows of ``w[g]`` are 32 gate rows followed by their 32 up rows
    (:func:`interleave_gate_up` builds that order); the result is ``silu(gate) * up`` with ``N / 2`` columns.
    """
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 3 or x.shape[1] != w.shape[2]:
        raise FusedGemmError(f"grouped_gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}")
    if not x.is_contiguous() or not w.is_contiguous():
        raise FusedGemmError("operands must be contiguous")
    G, N, K = w.shape
    if group_offsets.dtype != torch.int32 or group_offsets.numel() != G + 1 or not group_offsets.is_cuda or not group_offsets.is_contiguous():
        raise FusedGemmError("group_offsets must be a contiguous int32 device tensor with one entry more than there are groups")
    if G > MAX_GROUPS:
        raise FusedGemmError(f"at most {MAX_GROUPS} groups per call")
    R = x.shape[0]
    out_cols = N // 2 if act == "swiglu" else N
    if out is None:
        out = torch.empty(R, out_cols, dtype=torch.bfloat16, device=x.device)
    else:
        _check_out(out, R, out_cols)
    a = _Args()
    a.act = ACTS[act]
    a.A, a.B, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.M, a.N, a.K, a.rank, a.npes, a.mode = R, N, K, 0, 1, MODES["grouped"]
    a.epoch = 1
    a.group_offsets, a.groups = group_offsets.data_ptr(), G
    a.error_flag = _error_flag(x.device).data_ptr()
    _launch(a, torch.cuda.current_stream().cuda_stream)
    return out


def interleave_gate_up(w_gate_up: torch.Tensor) -> torch.Tensor:
    """``[..., 2F, K]`` with the F gate rows first and the F up rows after them -> the row order that
    ``grouped_gemm(..., act="swiglu")`` expects: blocks of 32 gate rows followed by the matching 32 up rows."""
    *lead, two_f, K = w_gate_up.shape
    F = two_f // 2
    if two_f % 64:
        raise FusedGemmError("the gate and up projections must each have a multiple of 32 rows")
    gate = w_gate_up[..., :F, :].reshape(*lead, F // 32, 32, K)
    up = w_gate_up[..., F:, :].reshape(*lead, F // 32, 32, K)
    return torch.stack((gate, up), dim=-3).reshape(*lead, two_f, K).contiguous()


class GemmReduceScatter:
    """Row-parallel GEMM fused with reduce-scatter (or all-reduce) over the world team.

    ``forward(x, w)``: ``x`` is ``[M, K_local]``, ``w`` ``[N, K_local]``; returns this rank's
    ``[M/npes, N]`` rows of the summed product (``mode="rs"``) or the whole ``[M, N]`` (``"ar"``).
    Without ``out=`` the output tensor is owned by the object and overwritten by the next call; with ``out=``
    (reduce-scatter only) the result is written there, e.g. straight into the shard of the next layer's
    all-gather buffer.

    ``use_multicast``: True = the switch path wherever the heap has a multicast window, False = the push path,
    None (default) = by team size: the switch path from four PEs on, the push path below.  With two or three PEs an
    owner adds only one or two partial tiles, which the push path's epilogue does faster than a trip through the
    switch (measured at 2 PEs: 0.33 ms push, 0.36 ms switch per 8192 x 8192 x 3584 GEMM); from four PEs on the owner's
    ingress and its epilogue work grow with the PE count on the push path and stay constant on the switch path.
    ``BSHMEM_FUSED_REDUCE_PATH=switch|push`` overrides the automatic choice.
    """

    def __init__(self, M: int, N: int, mode: str = "rs", wait_limit_ms: int = 0, use_multicast: bool | None = None):
        from .. import core
        self.core = core
        self.rank, self.npes = core.my_pe(), core.n_pes()
        if self.npes > MAX_PES:
            raise FusedGemmError(f"at most {MAX_PES} PEs")
        self.M, self.N, self.mode = M, N, mode
        self.wait_limit_ms = wait_limit_ms
        self.rows = M // self.npes
        self.epoch = 0
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        tiles = (self.rows // 128) * (N // 256)
        self.recv = self.flags = None
        self.switch_path = False
        self._stage_mc = self._out_mc = 0
        if mode == "ar" and self.npes > 1:
            self.out = core.tensor((M, N), torch.bfloat16)
        else:
            self.out = torch.empty(self.rows if mode == "rs" else M, N, dtype=torch.bfloat16, device=dev)
        self._peer = {}
        if use_multicast is None:
            forced = os.environ.get("BSHMEM_FUSED_REDUCE_PATH", "").lower()
            use_multicast = forced == "switch" or (forced != "push" and self.npes >= 4)
        if self.npes > 1:
            mc_ptr = H.load().nvshmemx_mc_ptr
            # Two generations of partial-tile storage by call parity: a fast peer may already be in call k+1.
            # With a multicast window it is one [M, N] staging buffer per generation that only its owner writes
            # (the tile owners read the sum of all PEs' copies through the switch); without one, receive slots
            # [npes, M/npes, N] that the peers push into.
            probe = core.tensor((2, M, N), torch.bfloat16)
            if use_multicast:
                self._stage_mc = int(mc_ptr(0, C.c_void_p(probe.data_ptr())) or 0)
                if mode == "ar":
                    self._out_mc = int(mc_ptr(0, C.c_void_p(self.out.data_ptr())) or 0)
            self.switch_path = bool(self._stage_mc) and (mode == "rs" or bool(self._out_mc))
            self.recv = probe  # the same bytes serve as staging buffer or as receive slots: 2 * M * N elements either way
            self.flags = core.tensor((self.npes * max(tiles, 1),), torch.int64, zero=True)
            for q in range(self.npes):
                self._peer[q] = (core.peer_ptr(self.recv, q), core.peer_ptr(self.flags, q), core.peer_ptr(self.out, q) if mode == "ar" else 0)
            core.barrier_all()
            torch.cuda.synchronize()

    def forward(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        _check_operands(x, w)
        if x.shape[0] != self.M or w.shape[0] != self.N:
            raise FusedGemmError("operand shapes differ from the ones this object was built for")
        if out is None:
            out = self.out
        elif self.mode != "rs":
            raise FusedGemmError("`out=` is for the reduce-scatter mode (the all-reduce output lives in symmetric memory)")
        else:
            _check_out(out, self.rows, self.N)
        self.epoch += 1
        a = _Args()
        a.A, a.B, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
        a.M, a.N, a.K, a.rank, a.npes, a.mode = self.M, self.N, x.shape[1], self.rank, self.npes, MODES[self.mode]
        a.epoch, a.wait_limit_ms = self.epoch, self.wait_limit_ms
        a.error_flag = _error_flag(self.device).data_ptr()
        if self.npes > 1:
            half = (self.epoch & 1) * self.M * self.N * 2
            a.flags_local = self.flags.data_ptr()
            if self.switch_path:
                a.stage_local = self.recv.data_ptr() + half
                a.stage_mc = self._stage_mc + half
            else:
                a.recv_local = self.recv.data_ptr() + half
            for q in range(self.npes):
                a.recv_peer[q] = self._peer[q][0] + half
                a.flags_peer[q] = self._peer[q][1]
                a.out_peer[q] = self._peer[q][2]
            a.out_mc = self._out_mc
        _launch(a, torch.cuda.current_stream().cuda_stream)
        if self.mode == "ar" and self.npes > 1:
            # Tiles written by the other PEs are complete once everyone's kernel has ended.
            self.core.barrier_all(stream=torch.cuda.current_stream())
        return out

    __call__ = forward

    def close(self) -> None:
        if self.npes > 1:
            torch.cuda.synchronize()
            self.core.free_tensor(self.recv)
            self.core.free_tensor(self.flags)
            if self.mode == "ar":
                self.core.free_tensor(self.out)
            self.recv = self.flags = None


class AllGatherGemm:
    """Column-parallel GEMM fused with the all-gather of its activations.

    Write this rank's ``[M/npes, K]`` shard into :attr:`shard` (a view of the symmetric gathered
    buffer), then ``forward(w)`` with ``w`` ``[N_local, K]`` returns ``[M, N_local]``.  A world sync
    is issued on the stream before each launch so that no peer overwrites a buffer still being read.

    ``copy_engine=False`` (default): two warps of every CTA of the GEMM kernel send the shard, so the transfer
    needs nothing but the kernel itself.  ``copy_engine=True`` (or ``BSHMEM_FUSED_AG_PATH=copy_engine``): the shard
    goes to the peers as one stream-ordered put with signal per peer (``nvshmemx_putmem_signal_on_stream``: a
    copy-engine copy and a flag write), nearest peer first, on a side stream that runs beside the GEMM kernel; no SM
    time is spent on the transfer and the calling stream waits for those copies after the kernel.  That path is the
    faster one on 2 PEs (0.36 ms against 0.44 ms at 8192 x 3584 x 8192) and passes the correctness tests on 8, but at
    the full size on 4 and 8 PEs, where CTAs of the GEMM start polling the flags while copies are still in
    flight, the flags did not arrive within the wait limit; until that is understood it is an option, not the default.
    """

    def __init__(self, M: int, K: int, wait_limit_ms: int = 0, copy_engine: bool | None = None, max_ctas: int = 0):
        from .. import core
        self.core = core
        self.rank, self.npes = core.my_pe(), core.n_pes()
        if self.npes > MAX_PES:
            raise FusedGemmError(f"at most {MAX_PES} PEs")
        self.M, self.K, self.wait_limit_ms = M, K, wait_limit_ms
        self.max_ctas = max_ctas  # 0: one CTA per SM; fewer leaves SMs to other work (every PE must pass the same value)
        self.rows = M // self.npes
        self.epoch = 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        if self.npes > 1:
            self.gathered = core.tensor((M, K), torch.bfloat16)
            self.flags = core.tensor((self.npes * max(self.rows // 128, 1),), torch.int64, zero=True)
            self._peer = {q: (core.peer_ptr(self.gathered, q), core.peer_ptr(self.flags, q)) for q in range(self.npes)}
            if copy_engine is None:
                copy_engine = os.environ.get("BSHMEM_FUSED_AG_PATH", "warps") == "copy_engine"
            self.copy_engine = copy_engine
            if copy_engine:
                self._comm = torch.cuda.Stream(device=self.device)
                self._ready, self._sent = torch.cuda.Event(), torch.cuda.Event()
            core.barrier_all()
            torch.cuda.synchronize()
        else:
            self.gathered = torch.empty(M, K, dtype=torch.bfloat16, device=self.device)
            self.flags = None
            self.copy_engine = False
        self.shard = self.gathered[self.rank * self.rows:(self.rank + 1) * self.rows]
        self.out = None

    def forward(self, w: torch.Tensor, out: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
        """``act(gathered @ w.T)``.  Without ``out=`` the result tensor is owned by the object and overwritten by the
        next call; ``act`` is None or ``"gelu_tanh"`` (fused into the epilogue)."""
        _check_operands(self.gathered, w)
        N = w.shape[0]
        if out is None:
            if self.out is None or self.out.shape[1] != N:
                self.out = torch.empty(self.M, N, dtype=torch.bfloat16, device=self.device)
            out = self.out
        else:
            _check_out(out, self.M, N)
        self.epoch += 1
        a = _Args()
        a.act = ACTS[act]
        a.A, a.B, a.out = self.gathered.data_ptr(), w.data_ptr(), out.data_ptr()
        a.M, a.N, a.K, a.rank, a.npes, a.mode = self.M, N, self.K, self.rank, self.npes, MODES["ag"]
        a.epoch, a.wait_limit_ms, a.max_ctas = self.epoch, self.wait_limit_ms, self.max_ctas
        a.error_flag = _error_flag(self.device).data_ptr()
        if self.npes > 1:
            a.ag_flags_local = self.flags.data_ptr()
            for q in range(self.npes):
                a.ag_peer[q] = self._peer[q][0]
                a.ag_flags_peer[q] = self._peer[q][1]
            self.core.sync_all()  # every rank has finished reading the previous gathered buffer
            if self.copy_engine:
                a.ag_external = 1
                main = torch.cuda.current_stream()
                self._ready.record(main)
                self._comm.wait_event(self._ready)
                lib = H.load()
                tmr = max(self.rows // 128, 1)
                shard_ptr, shard_bytes = self.shard.data_ptr(), self.rows * self.K * 2
                flag_ptr = self.flags.data_ptr() + 8 * self.rank * tmr
                for o in range(1, self.npes):
                    # the same symmetric addresses on the peer: its slot for my shard, its flag for my shard
                    lib.nvshmemx_putmem_signal_on_stream(C.c_void_p(shard_ptr), C.c_void_p(shard_ptr), shard_bytes, C.c_void_p(flag_ptr), self.epoch, 9,
                                                         (self.rank + o) % self.npes, C.c_void_p(self._comm.cuda_stream))
                self._sent.record(self._comm)
        _launch(a, torch.cuda.current_stream().cuda_stream)
        if self.npes > 1 and self.copy_engine:
            torch.cuda.current_stream().wait_event(self._sent)  # the shard may be rewritten once the copies have read it
        return out

    __call__ = forward

    def close(self) -> None:
        if self.npes > 1:
            torch.cuda.synchronize()
            self.core.free_tensor(self.gathered)
            self.core.free_tensor(self.flags)
            self.gathered = self.flags = None
