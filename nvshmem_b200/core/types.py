"""Enumerations, exceptions and the stream wrapper of the Python layer
(reference: nvshmem4py/nvshmem/core/nvshmem_types.py, _internal_tracking.py)."""
from __future__ import annotations

import enum


class NvshmemError(RuntimeError):
    """A library call failed; the message names the call and the status code."""


class NvshmemInvalid(ValueError):
    """An argument is not usable (wrong dtype, non-symmetric tensor, bad team ...)."""


class ComparisonType(enum.IntEnum):
    CMP_EQ = 0
    CMP_NE = 1
    CMP_GT = 2
    CMP_LE = 3
    CMP_LT = 4
    CMP_GE = 5


class SignalOp(enum.IntEnum):
    SIGNAL_SET = 9
    SIGNAL_ADD = 10


class BufferKind(enum.IntEnum):
    NORMAL = 0
    PEER = 1
    MULTIMEM = 2
    EXTERNAL = 3


class NvshmemStream:
    """Anything with a CUDA stream handle: a ``torch.cuda.Stream``, an int, or None
    (the current torch stream)."""

    def __init__(self, stream=None):
        self._stream = stream

    @property
    def handle(self) -> int:
        return stream_handle(self._stream)


def stream_handle(stream) -> int:
    if stream is None:
        import torch
        return int(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else 0
    if isinstance(stream, NvshmemStream):
        return stream.handle
    if isinstance(stream, int):
        return stream
    for attr in ("cuda_stream", "handle", "ptr"):
        if hasattr(stream, attr):
            return int(getattr(stream, attr))
    raise NvshmemInvalid(f"cannot take a CUDA stream from {type(stream).__name__}")
