"""Symmetric memory as Python objects and torch tensors
(reference: nvshmem4py/nvshmem/core/memory.py, nvshmem_types.py NvshmemResource, interop/torch.py).

A :class:`Buffer` is a span of the symmetric heap.  Every buffer handed out is
tracked with a reference count and a kind (normal, peer view, multicast view,
external); freeing is explicit and collective, as in nvshmem4py: a buffer that
is garbage-collected without ``free`` is reported, not silently released, since
a unilateral release would break the symmetry of the heap.
"""
from __future__ import annotations

import ctypes as C
import math
import warnings

from ..bindings import host as H
from .types import BufferKind, NvshmemError, NvshmemInvalid

_tracked: dict[int, dict] = {}  # ptr -> {buffer, ref_count, kind, freed}: allocations (NORMAL) and registered ranges (EXTERNAL)
# Views (peer and multicast aliases) are counted apart from allocations, keyed by (address, kind): the view of
# the calling PE itself has the allocation's own address and must never touch the allocation's record.
_views: dict[tuple[int, int], dict] = {}


class Buffer:
    """A span of device (or, with the host heap, host) memory; exposes the CUDA array interface."""

    def __init__(self, ptr: int, size: int, kind: BufferKind = BufferKind.NORMAL, device_memory: bool = True, owner=None):
        self.ptr = int(ptr)
        self.size = int(size)
        self.kind = kind
        self.device_memory = device_memory
        self._owner = owner  # keeps a parent buffer alive for peer / multicast views

    @property
    def handle(self) -> int:
        return self.ptr

    @property
    def __cuda_array_interface__(self):
        if not self.device_memory:
            raise AttributeError("host-heap buffers are not CUDA arrays")
        return {"shape": (self.size,), "typestr": "|u1", "data": (self.ptr, False), "version": 3, "strides": None}

    def __repr__(self):
        return f"Buffer(ptr={self.ptr:#x}, size={self.size}, kind={self.kind.name})"


def _gpu_backend() -> bool:
    return H.load().nvshmemx_b200_heap_info(7) != 0


def buffer(size: int, alignment: int = 0, zero: bool = False) -> Buffer:
    """Collective: allocates `size` bytes of symmetric memory on every PE."""
    lib = H.load()
    if size <= 0:
        raise NvshmemInvalid("buffer size must be positive")
    if zero:
        ptr = lib.nvshmem_calloc(size, 1)
    elif alignment:
        ptr = lib.nvshmem_align(alignment, size)
    else:
        ptr = lib.nvshmem_malloc(size)
    if not ptr:
        raise NvshmemError(f"symmetric allocation of {size} bytes failed")
    buf = Buffer(ptr, size, BufferKind.NORMAL, _gpu_backend())
    _tracked[ptr] = {"buffer": buf, "ref_count": 1, "kind": BufferKind.NORMAL, "freed": False}
    return buf


def free(buf: Buffer) -> None:
    """Collective: returns a buffer obtained from :func:`buffer`.  Freeing a view (peer, multicast) only drops the
    view's own reference and never touches the allocation it aliases (as in nvshmem4py)."""
    if buf.kind in (BufferKind.PEER, BufferKind.MULTIMEM):
        key = (buf.ptr, int(buf.kind))
        rec = _views.get(key)
        if rec is None:
            raise NvshmemInvalid(f"{buf!r} is not a live view")
        rec["ref_count"] -= 1
        if rec["ref_count"] <= 0:
            del _views[key]
        return
    rec = _tracked.get(buf.ptr)
    if rec is None or rec["freed"]:
        raise NvshmemInvalid(f"{buf!r} is not a live symmetric buffer")
    rec["ref_count"] -= 1
    if rec["ref_count"] > 0:
        return
    rec["freed"] = True
    del _tracked[buf.ptr]
    if rec["kind"] == BufferKind.NORMAL:
        H.load().nvshmem_free(C.c_void_p(buf.ptr))


def _free_all_tracked() -> None:
    """Called by finalize: releases whatever the program left allocated, in allocation order."""
    for ptr in sorted(p for p, r in _tracked.items() if r["kind"] == BufferKind.NORMAL and not r["freed"]):
        H.load().nvshmem_free(C.c_void_p(ptr))
    _tracked.clear()
    _views.clear()


def get_peer_buffer(buf: Buffer, pe: int) -> Buffer:
    """This PE's mapping of the same buffer on PE `pe` (load/store reachable over NVLink)."""
    ptr = H.load().nvshmem_ptr(C.c_void_p(buf.ptr), int(pe))
    if not ptr:
        raise NvshmemInvalid(f"{buf!r} is not symmetric or PE {pe} is out of range")
    view = Buffer(ptr, buf.size, BufferKind.PEER, buf.device_memory, owner=buf)
    rec = _views.setdefault((ptr, int(BufferKind.PEER)), {"buffer": view, "ref_count": 0})
    rec["ref_count"] += 1
    return view


def get_multicast_buffer(team: int, buf: Buffer) -> Buffer:
    """The NVLink-multicast alias of `buf` for `team` (stores reach every member, ld_reduce sums over them)."""
    ptr = H.load().nvshmemx_mc_ptr(int(team), C.c_void_p(buf.ptr))
    if not ptr:
        raise NvshmemInvalid("no multicast mapping: NVLS is unavailable or the team does not span the multicast group")
    view = Buffer(ptr, buf.size, BufferKind.MULTIMEM, True, owner=buf)
    rec = _views.setdefault((ptr, int(BufferKind.MULTIMEM)), {"buffer": view, "ref_count": 0})
    rec["ref_count"] += 1
    return view


def register_external_buffer(buf, size: int | None = None) -> Buffer:
    """Collective: maps caller-owned device memory into the symmetric heap and returns the symmetric view.

    `buf` is a :class:`Buffer`, an int address or anything with ``data_ptr()`` / ``nbytes``.  The memory must be one
    ``cuMemCreate`` allocation of this GPU, shareable as a POSIX file descriptor, whose size is a multiple of the heap's
    growth granule (512 MB by default) and the same on every PE: memory from ``cudaMalloc`` or torch's default allocator
    does not qualify (reference: nvshmem4py/nvshmem/core/memory.py, register_external_buffer; the reference's
    torch_mempool example allocates such memory through a pluggable allocator).
    """
    if isinstance(buf, Buffer):
        ptr, nbytes = buf.ptr, buf.size
    elif hasattr(buf, "data_ptr"):
        ptr, nbytes = int(buf.data_ptr()), int(buf.numel() * buf.element_size())
    else:
        ptr, nbytes = int(buf), size
    if size is not None:
        nbytes = int(size)
    if not nbytes:
        raise NvshmemInvalid("register_external_buffer needs the size of the allocation")
    lib = H.load()
    lib.nvshmemx_buffer_register_symmetric.restype = C.c_void_p
    lib.nvshmemx_buffer_register_symmetric.argtypes = [C.c_void_p, C.c_size_t, C.c_int]
    mapped = lib.nvshmemx_buffer_register_symmetric(C.c_void_p(ptr), nbytes, 0)
    if not mapped:
        raise NvshmemError("the buffer cannot be registered: it must be a cuMemCreate allocation of this GPU with a POSIX-FD handle type "
                           "and a size that is a multiple of the heap's growth granule")
    view = Buffer(mapped, nbytes, BufferKind.EXTERNAL, True, owner=buf)
    _tracked[mapped] = {"buffer": view, "ref_count": 1, "kind": BufferKind.EXTERNAL, "freed": False}
    return view


def unregister_external_buffer(view: Buffer) -> None:
    """Collective: undoes :func:`register_external_buffer`."""
    lib = H.load()
    lib.nvshmemx_buffer_unregister_symmetric.restype = C.c_int
    lib.nvshmemx_buffer_unregister_symmetric.argtypes = [C.c_void_p, C.c_size_t]
    if lib.nvshmemx_buffer_unregister_symmetric(C.c_void_p(view.ptr), view.size) != 0:
        raise NvshmemInvalid(f"{view!r} was not made by register_external_buffer")
    _tracked.pop(view.ptr, None)


# ------------------------------------------------------------------ torch interop
_DTYPE_SIZE = None


def _as_torch(buf: Buffer, shape, dtype):
    import torch
    if buf.device_memory:
        flat = torch.as_tensor(buf, device=f"cuda:{torch.cuda.current_device()}")
    else:
        flat = torch.frombuffer((C.c_uint8 * buf.size).from_address(buf.ptr), dtype=torch.uint8)
    nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
    t = flat[:nbytes].view(dtype).view(*shape)
    t._bshmem_buffer = buf  # the tensor aliases the buffer; the buffer must outlive it
    return t


def tensor(shape, dtype=None, zero: bool = False):
    """Collective: a torch tensor backed by symmetric memory (same shape and dtype on every PE)."""
    import torch
    dtype = dtype or torch.float32
    shape = tuple(int(s) for s in (shape if hasattr(shape, "__iter__") else (shape,)))
    nbytes = max(1, math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    return _as_torch(buffer(nbytes, zero=zero), shape, dtype)


def bytetensor(shape, dtype=None):
    import torch
    return tensor(shape, torch.uint8)


def _buffer_of(t) -> Buffer:
    buf = getattr(t, "_bshmem_buffer", None)
    if buf is None:
        # A view of a symmetric tensor: find the allocation that contains it.
        ptr = t.data_ptr()
        for base, rec in _tracked.items():
            if base <= ptr < base + rec["buffer"].size:
                return Buffer(ptr, rec["buffer"].size - (ptr - base), rec["kind"], rec["buffer"].device_memory, owner=rec["buffer"])
        raise NvshmemInvalid("the tensor is not backed by symmetric memory (allocate it with nvshmem_b200.core.tensor)")
    return buf


def tensor_ptr(t) -> int:
    """Address of a symmetric tensor, checked."""
    _buffer_of(t)
    return int(t.data_ptr())


def peer_ptr(t, pe: int) -> int:
    """Address at which PE `pe`'s copy of symmetric tensor `t` is mapped in this process."""
    ptr = H.load().nvshmem_ptr(C.c_void_p(int(t.data_ptr())), int(pe))
    if not ptr:
        raise NvshmemInvalid("not a symmetric tensor or PE out of range")
    return int(ptr)


def free_tensor(t) -> None:
    """Collective: frees a tensor made by :func:`tensor`.  The tensor must not be used afterwards."""
    buf = getattr(t, "_bshmem_buffer", None)
    if buf is None:
        raise NvshmemInvalid("free_tensor needs the tensor returned by tensor(), not a view of it")
    free(buf)


def get_peer_tensor(t, pe: int):
    """PE `pe`'s copy of `t`, as a tensor on this device.  Meant for this library's kernels and
    for copies; do not hand it to library GEMM or attention kernels as an operand."""
    view = get_peer_buffer(_buffer_of(t), pe)
    return _as_torch(view, tuple(t.shape), t.dtype)


def get_multicast_tensor(team: int, t):
    view = get_multicast_buffer(team, _buffer_of(t))
    return _as_torch(view, tuple(t.shape), t.dtype)


def register_external_tensor(t):
    return register_external_buffer(t)
