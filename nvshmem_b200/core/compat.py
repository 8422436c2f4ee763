"""Remaining public names of the reference's Python package, so that code written against
``nvshmem.core`` finds them here too (reference: nvshmem4py/nvshmem/core/nvshmem_types.py, utils.py,
direct.py, init_fini.py, teams.py, interop/torch.py, interop/cupy.py)."""
from __future__ import annotations

import ctypes as C
import enum
import warnings

from ..bindings import host as H
from . import memory as _memory
from .types import BufferKind, NvshmemError, NvshmemInvalid

UniqueID = H.UniqueId
TeamConfig = H.TeamConfig
BufferTypes = BufferKind


class TeamUniqueId(int):
    """The 64-bit id that `team_init` members agree on (see `get_team_unique_id`)."""


class InitStatus(enum.IntEnum):
    STATUS_NOT_INITIALIZED = 0
    STATUS_IS_BOOTSTRAPPED = 1
    STATUS_IS_INITIALIZED = 2
    STATUS_LIMITED_MPG = 3
    STATUS_FULL_MPG = 4
    STATUS_INVALID = 0x7FFFFFFF


class NvshmemStreamsType(enum.IntEnum):
    """Which stream an operation is ordered on when the caller passes none."""
    DEFAULT = 0
    CURRENT = 1


class NvshmemWarning(UserWarning):
    pass


class MutableEnum:
    """A namespace of named integer constants that can grow at run time (team handles are added to it)."""

    def __init__(self, **members):
        self.__dict__.update(members)

    def add(self, name: str, value: int) -> None:
        setattr(self, name, int(value))

    def __contains__(self, name) -> bool:
        return name in self.__dict__

    def __iter__(self):
        return iter(self.__dict__.items())


class Version:
    def __init__(self, openshmem_spec_version="", nvshmem4py_version="", libnvshmem_version=""):
        self.openshmem_spec_version = openshmem_spec_version
        self.nvshmem4py_version = nvshmem4py_version
        self.libnvshmem_version = libnvshmem_version

    def __repr__(self):
        return (f"bshmem Python layer:\n    library version: {self.libnvshmem_version}\n"
                f"    OpenSHMEM spec version: {self.openshmem_spec_version}\n    Python layer version: {self.nvshmem4py_version}\n")


class NvshmemKernelObject:
    """A loaded device-code object (CUmodule or CUlibrary handle) that carries a copy of the device state.
    Build it with :meth:`from_handle`; pass it to ``module_init`` / ``library_init`` before launching its kernels."""

    def __new__(cls, *args, **kwargs):
        raise RuntimeError("NvshmemKernelObject cannot be instantiated directly; use NvshmemKernelObject.from_handle")

    @classmethod
    def _make(cls, handle: int):
        self = object.__new__(cls)
        self.handle = int(handle)
        return self

    @staticmethod
    def from_handle(handle) -> "NvshmemKernelObject":
        return NvshmemKernelObject._make(int(handle))

    @staticmethod
    def from_obj(obj) -> "NvshmemKernelObject":
        """From an object that exposes its driver handle as ``.handle`` (e.g. a cuda.core ObjectCode)."""
        return NvshmemKernelObject._make(int(getattr(obj, "handle")))

    def __int__(self) -> int:
        return self.handle


class NvshmemResource:
    """Memory resource over the symmetric heap: ``allocate`` / ``deallocate`` in the style of cuda.core's
    MemoryResource, backed by the same tracked buffers as :func:`nvshmem_b200.core.buffer`."""

    def __init__(self, device=None):
        self.device = device

    def allocate(self, size: int, stream=None):
        return _memory.buffer(size)

    def deallocate(self, ptr, size: int = 0, stream=None) -> None:
        rec = _memory._tracked.get(int(getattr(ptr, "ptr", ptr)))
        if rec is None:
            raise NvshmemInvalid("not a buffer of the symmetric heap")
        _memory.free(rec["buffer"])

    @property
    def is_device_accessible(self) -> bool:
        return True

    @property
    def is_host_accessible(self) -> bool:
        return not _memory._gpu_backend()

    @property
    def device_id(self) -> int:
        dev = int(H.load().nvshmemx_b200_heap_info(8))
        return dev - (1 << 64) if dev >= (1 << 63) else dev  # -1 on the host-memory back end


def module_finalize(mod) -> None:
    st = H.load().nvshmemx_cumodule_finalize(C.c_void_p(int(mod)))
    if st != 0:
        raise NvshmemError(f"nvshmemx_cumodule_finalize failed with status {st}")


def library_finalize(lib) -> None:
    # A CUlibrary holds no library-side resources here: its device-state copy simply stops being refreshed.
    return None


def dtype_nbytes(dtype) -> int:
    """Size in bytes of one element of a torch / numpy dtype."""
    try:
        import torch
        if isinstance(dtype, torch.dtype):
            return torch.empty((), dtype=dtype).element_size()
    except ImportError:
        pass
    import numpy as np
    return int(np.dtype(dtype).itemsize)


def get_size(shape, dtype) -> int:
    """Bytes needed for an array of `shape` and `dtype`."""
    n = 1
    for d in (shape if hasattr(shape, "__iter__") else (shape,)):
        n *= int(d)
    return n * dtype_nbytes(dtype)


# ------------------------------------------------------------------ torch interop additions
def tensor_get_buffer(t) -> _memory.Buffer:
    """The tracked buffer behind a tensor made by ``tensor()`` (or a view of one that starts at its base)."""
    buf = getattr(t, "_bshmem_buffer", None)
    if buf is None:
        rec = _memory._tracked.get(int(t.data_ptr()))
        if rec is None:
            raise NvshmemInvalid("the tensor does not start at a symmetric allocation")
        buf = rec["buffer"]
    return buf


def unregister_external_tensor(t) -> None:
    _memory.unregister_external_buffer(tensor_get_buffer(t))


# ------------------------------------------------------------------ cupy interop (only where cupy is installed)
def _cupy():
    try:
        import cupy
        return cupy
    except ImportError as e:
        raise NvshmemError("cupy is not installed in this environment; use the torch interop (tensor, bytetensor, ...)") from e


def array(shape, dtype="float32"):
    cp = _cupy()
    buf = _memory.buffer(get_size(shape, dtype))
    mem = cp.cuda.UnownedMemory(buf.ptr, buf.size, buf)
    out = cp.ndarray(shape, dtype=dtype, memptr=cp.cuda.MemoryPointer(mem, 0))
    out._bshmem_buffer = buf
    return out


def bytearray(shape):
    return array(shape, "uint8")


def array_get_buffer(a) -> _memory.Buffer:
    buf = getattr(a, "_bshmem_buffer", None)
    if buf is None:
        raise NvshmemInvalid("not an array made by array()")
    return buf


def free_array(a) -> None:
    _memory.free(array_get_buffer(a))


def _array_view(buf: _memory.Buffer, like):
    cp = _cupy()
    mem = cp.cuda.UnownedMemory(buf.ptr, buf.size, buf)
    return cp.ndarray(like.shape, dtype=like.dtype, memptr=cp.cuda.MemoryPointer(mem, 0))


def get_peer_array(a, pe: int):
    return _array_view(_memory.get_peer_buffer(array_get_buffer(a), pe), a)


def get_multicast_array(team: int, a):
    return _array_view(_memory.get_multicast_buffer(team, array_get_buffer(a)), a)


def register_external_array(a):
    return _array_view(_memory.register_external_buffer(int(a.data.ptr), int(a.nbytes)), a)


def unregister_external_array(a) -> None:
    rec = _memory._tracked.get(int(a.data.ptr))
    if rec is None:
        raise NvshmemInvalid("not a registered array")
    _memory.unregister_external_buffer(rec["buffer"])


def warn(msg: str) -> None:
    warnings.warn(msg, NvshmemWarning, stacklevel=2)
