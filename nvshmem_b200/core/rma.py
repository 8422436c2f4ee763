"""Host-initiated, stream-ordered RMA on symmetric tensors
(reference: nvshmem4py/nvshmem/core/rma.py: on-stream only)."""
from __future__ import annotations

import ctypes as C

from ..bindings import host as H
from .memory import tensor_ptr
from .types import ComparisonType, NvshmemInvalid, SignalOp, stream_handle


def _nbytes(t) -> int:
    return t.numel() * t.element_size()


def _check_pair(dst, src):
    if _nbytes(dst) < _nbytes(src):
        raise NvshmemInvalid("destination is smaller than source")
    if not dst.is_contiguous() or not src.is_contiguous():
        raise NvshmemInvalid("put/get need contiguous tensors")


def put(dst, src, remote_pe: int, stream=None) -> None:
    """Copies local `src` into `dst` on `remote_pe` (`dst` symmetric), ordered on `stream`."""
    _check_pair(dst, src)
    H.load().nvshmemx_putmem_on_stream(C.c_void_p(tensor_ptr(dst)), C.c_void_p(src.data_ptr()), _nbytes(src), int(remote_pe), C.c_void_p(stream_handle(stream)))


def get(dst, src, remote_pe: int, stream=None) -> None:
    """Copies `src` on `remote_pe` (`src` symmetric) into local `dst`."""
    _check_pair(dst, src)
    H.load().nvshmemx_getmem_on_stream(C.c_void_p(dst.data_ptr()), C.c_void_p(tensor_ptr(src)), _nbytes(src), int(remote_pe), C.c_void_p(stream_handle(stream)))


def put_signal(dst, src, signal_var, signal_val: int, signal_op: SignalOp, remote_pe: int, stream=None) -> None:
    """put followed by a signal update on `remote_pe` that becomes visible after the data."""
    _check_pair(dst, src)
    H.load().nvshmemx_putmem_signal_on_stream(C.c_void_p(tensor_ptr(dst)), C.c_void_p(src.data_ptr()), _nbytes(src), C.c_void_p(tensor_ptr(signal_var)),
                                             int(signal_val), int(signal_op), int(remote_pe), C.c_void_p(stream_handle(stream)))


def signal_op(signal_var, signal_val: int, signal_op: SignalOp, remote_pe: int, stream=None) -> None:
    H.load().nvshmemx_signal_op_on_stream(C.c_void_p(tensor_ptr(signal_var)), int(signal_val), int(signal_op), int(remote_pe), C.c_void_p(stream_handle(stream)))


def signal_wait(signal_var, signal_val: int, signal_op: ComparisonType = ComparisonType.CMP_GE, stream=None) -> None:
    """Blocks `stream` until the local signal word satisfies the comparison."""
    H.load().nvshmemx_signal_wait_until_on_stream(C.c_void_p(tensor_ptr(signal_var)), int(signal_op), int(signal_val), C.c_void_p(stream_handle(stream)))


def signal_fetch(signal_var) -> int:
    return int(H.load().nvshmem_signal_fetch(C.c_void_p(tensor_ptr(signal_var))))


def quiet(stream=None) -> None:
    H.load().nvshmemx_quiet_on_stream(C.c_void_p(stream_handle(stream)))
