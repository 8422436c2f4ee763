"""Stream-ordered collectives on symmetric tensors
(reference: nvshmem4py/nvshmem/core/collective.py)."""
from __future__ import annotations

import ctypes as C

from ..bindings import host as H
from .memory import tensor_ptr
from .types import NvshmemError, NvshmemInvalid, stream_handle

_OPS = {"and": H.OP_AND, "or": H.OP_OR, "xor": H.OP_XOR, "min": H.OP_MIN, "max": H.OP_MAX, "sum": H.OP_SUM, "prod": H.OP_PROD}
REDUCE_ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls_oneshot": 3, "nvls_twoshot": 4, "ll": 5, "ll128": 6, "recexch": 7}
FCOLLECT_ALGOS = {"auto": 0, "push": 1, "ll": 2, "nvls": 3, "ll128": 4}
RS_ALGOS = {"auto": 0, "pull": 1, "nvls": 2}
BCAST_ALGOS = {"auto": 0, "push": 1, "ll": 2, "nvls": 3, "pull": 4}


def _dtype_code(t) -> int:
    import torch
    table = {torch.int8: H.DT_I8, torch.uint8: H.DT_U8, torch.int16: H.DT_I16, torch.int32: H.DT_I32, torch.int64: H.DT_I64, torch.float16: H.DT_F16,
             torch.bfloat16: H.DT_BF16, torch.float32: H.DT_F32, torch.float64: H.DT_F64}
    for name, code in (("uint16", H.DT_U16), ("uint32", H.DT_U32), ("uint64", H.DT_U64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = code
    if t.dtype not in table:
        raise NvshmemInvalid(f"dtype {t.dtype} is not supported by the collectives")
    return table[t.dtype]


def _check(st: int, what: str) -> None:
    if st != 0:
        raise NvshmemError(f"{what} failed with status {st}")


def reduce(team: int, dst, src, op: str = "sum", stream=None, algo: str = "auto") -> None:
    """All-reduce: dst = op over the team's members of src (element-wise).  In place is allowed."""
    if dst.numel() < src.numel() or dst.dtype != src.dtype:
        raise NvshmemInvalid("reduce: dst must have src's dtype and at least its size")
    _check(H.load().nvshmemx_b200_reduce_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), src.numel(), _dtype_code(src), _OPS[op],
                                                   REDUCE_ALGOS[algo], C.c_void_p(stream_handle(stream))), "reduce")


def reducescatter(team: int, dst, src, op: str = "sum", stream=None, algo: str = "auto") -> None:
    """dst[i] = op over members of src[my_pe*len(dst) + i]; src holds team_size * len(dst) elements."""
    if dst.dtype != src.dtype:
        raise NvshmemInvalid("reducescatter: dtype mismatch")
    _check(H.load().nvshmemx_b200_reducescatter_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), dst.numel(), _dtype_code(src),
                                                          _OPS[op], RS_ALGOS[algo], C.c_void_p(stream_handle(stream))), "reducescatter")


def fcollect(team: int, dst, src, stream=None, algo: str = "auto") -> None:
    """All-gather: member m's src lands at dst[m*len(src) : (m+1)*len(src)] on every member."""
    nbytes = src.numel() * src.element_size()
    _check(H.load().nvshmemx_b200_fcollect_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), nbytes, FCOLLECT_ALGOS[algo],
                                                     C.c_void_p(stream_handle(stream))), "fcollect")


def alltoall(team: int, dst, src, stream=None) -> None:
    """Block p of src goes to block my_pe of dst on member p; blocks are len(src)/team_size elements."""
    n = H.load().nvshmem_team_n_pes(int(team))
    nbytes = src.numel() * src.element_size() // max(n, 1)
    _check(H.load().nvshmemx_alltoallmem_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), nbytes, C.c_void_p(stream_handle(stream))),
           "alltoall")


def broadcast(team: int, dst, src, root: int = 0, stream=None, algo: str = "auto") -> None:
    nbytes = src.numel() * src.element_size()
    _check(H.load().nvshmemx_b200_broadcast_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), nbytes, int(root), BCAST_ALGOS[algo],
                                                      C.c_void_p(stream_handle(stream))), "broadcast")


def maxloc(team: int, dst, src, stream=None) -> None:
    """(value, index) pair with the largest value over the team; tensors are float64[2]."""
    _check(H.load().nvshmemx_double2_maxloc_reduce_on_stream(int(team), C.c_void_p(tensor_ptr(dst)), C.c_void_p(tensor_ptr(src)), 1, C.c_void_p(stream_handle(stream))),
           "maxloc")


def barrier(team: int, stream=None) -> None:
    _check(H.load().nvshmemx_barrier_on_stream(int(team), C.c_void_p(stream_handle(stream))), "barrier")


def barrier_all(stream=None) -> None:
    H.load().nvshmemx_barrier_all_on_stream(C.c_void_p(stream_handle(stream)))


def sync(team: int, stream=None) -> None:
    _check(H.load().nvshmemx_team_sync_on_stream(int(team), C.c_void_p(stream_handle(stream))), "sync")


def sync_all(stream=None) -> None:
    H.load().nvshmemx_sync_all_on_stream(C.c_void_p(stream_handle(stream)))


def collective_on_buffer(coll: str, team: int, dst, src, dtype: str | None = None, op: str | None = None, root: int = 0, stream=None, enable_timing: bool = False):
    """Name-driven entry (``coll`` in reduce, reducescatter, alltoall, fcollect, broadcast); returns the
    elapsed milliseconds when ``enable_timing`` is set, measured with CUDA events on `stream`."""
    import torch
    start = end = None
    if enable_timing:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(torch.cuda.current_stream() if stream is None else stream)
    if coll == "reduce":
        reduce(team, dst, src, op or "sum", stream)
    elif coll == "reducescatter":
        reducescatter(team, dst, src, op or "sum", stream)
    elif coll == "alltoall":
        alltoall(team, dst, src, stream)
    elif coll == "fcollect":
        fcollect(team, dst, src, stream)
    elif coll == "broadcast":
        broadcast(team, dst, src, root, stream)
    else:
        raise NvshmemInvalid(f"unknown collective {coll}")
    if enable_timing:
        end.record(torch.cuda.current_stream() if stream is None else stream)
        end.synchronize()
        return start.elapsed_time(end)
    return None
