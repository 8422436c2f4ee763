"""Initialisation and shutdown (reference: nvshmem4py/nvshmem/core/init_fini.py).

``init`` takes the unique id made by ``get_unique_id`` on one rank and shared
out of band.  The torch-idiomatic route is ``init(initializer_method="torch")``
(or ``uid=None`` with an initialised ``torch.distributed`` group): rank 0 makes
the id and broadcasts it through the process group.
"""
from __future__ import annotations

import atexit
import ctypes as C
import os

from ..bindings import host as H
from .types import NvshmemError, NvshmemInvalid

_initialized = False


def get_version() -> dict:
    lib = H.load()
    major, minor, patch = C.c_int(), C.c_int(), C.c_int()
    lib.nvshmem_info_get_version(C.byref(major), C.byref(minor))
    spec = (major.value, minor.value)
    lib.nvshmemx_vendor_get_version_info(C.byref(major), C.byref(minor), C.byref(patch))
    name = C.create_string_buffer(256)
    lib.nvshmem_info_get_name(name)
    return {"openshmem_spec_version": spec, "libnvshmem_version": (major.value, minor.value, patch.value), "name": name.value.decode()}


def get_unique_id(empty: bool = False) -> H.UniqueId:
    """Returns a unique id; with ``empty=True`` only the container (for ranks that will receive one)."""
    uid = H.UniqueId()
    if not empty:
        st = H.load().nvshmemx_get_uniqueid(C.byref(uid))
        if st != 0:
            raise NvshmemError(f"nvshmemx_get_uniqueid failed with status {st}")
    return uid


def _device_ordinal(device) -> int:
    """CUDA ordinal of `device`: an int, a ``torch.device``, a ``cuda.core`` Device (``device_id``), a CuPy device
    (``id``); -1 (the current device, or none with the host heap) for None and for a torch CPU device."""
    if device is None:
        return -1
    if isinstance(device, int):
        return device
    if hasattr(device, "type"):  # torch.device
        return device.index if device.type == "cuda" and device.index is not None else -1
    for attr in ("device_id", "id", "index"):
        v = getattr(device, attr, None)
        if isinstance(v, int):
            return v
    return int(device)


def _init_with_mpi(mpi_comm, dev: int) -> None:
    """Initialises over MPI (the bootstrap plugin opens the MPI library that is in the process).  `mpi_comm` is an
    mpi4py communicator, a ctypes object holding an ``MPI_Comm``, the integer address of one, or None for mpi4py's
    ``COMM_WORLD`` (reference: nvshmem4py/nvshmem/core/init_fini.py, initializer_method="mpi")."""
    from ..bindings import nvshmem as flat
    keep = None
    if mpi_comm is None:
        try:
            from mpi4py import MPI
        except ImportError as e:
            raise NvshmemInvalid("initializer_method='mpi' without a communicator needs mpi4py") from e
        mpi_comm = MPI.COMM_WORLD
    if isinstance(mpi_comm, int):
        addr = mpi_comm
    elif isinstance(mpi_comm, (C._SimpleCData, C.Structure)):
        addr, keep = C.addressof(mpi_comm), mpi_comm
    else:
        try:
            from mpi4py import MPI
            addr, keep = MPI._addressof(mpi_comm), mpi_comm
        except (ImportError, TypeError) as e:
            raise NvshmemInvalid(f"cannot take the address of the MPI communicator in {type(mpi_comm).__name__}") from e
    attr = flat.InitAttr()
    flat.set_attr_mpi_comm_args(addr, attr.ptr)
    attr._data["args"][0].view("int32")[8] = dev  # nvshmemx_init_args_t::cuda_device_id
    try:
        flat.hostlib_init_attr(flat.Flags.INIT_WITH_MPI_COMM, attr.ptr)
    except flat.NVSHMEMError as e:
        raise NvshmemError(f"initialisation over MPI failed with status {e.status}") from e
    del keep


def _uid_via_torch(rank: int, group=None) -> H.UniqueId:
    import torch
    import torch.distributed as dist
    payload = [get_unique_id().to_bytes() if rank == 0 else None]
    dist.broadcast_object_list(payload, src=0, group=group)
    return H.UniqueId.from_bytes(payload[0])


def init(device=None, uid: H.UniqueId | bytes | None = None, rank: int | None = None, nranks: int | None = None, mpi_comm=None,
         initializer_method: str = "uid") -> None:
    """Initialises the library for this process.

    device: CUDA ordinal, ``torch.device`` or None (current device; no GPU needed with the host heap).
    uid/rank/nranks: as returned by ``get_unique_id`` and the launcher.  With
    ``initializer_method="torch"`` they come from ``torch.distributed``.
    """
    global _initialized
    if _initialized:
        return
    if initializer_method == "emulated_mpi":
        raise NvshmemInvalid("initializer_method='emulated_mpi' is not offered; use 'mpi', 'uid' or 'torch'")
    if mpi_comm is not None or initializer_method == "mpi":
        _init_with_mpi(mpi_comm, _device_ordinal(device))
        _initialized = True
        atexit.register(finalize)
        return
    lib = H.load()
    if initializer_method == "torch" or uid is None:
        import torch.distributed as dist
        if not dist.is_initialized():
            raise NvshmemInvalid("init without a unique id needs an initialised torch.distributed process group")
        rank, nranks = dist.get_rank(), dist.get_world_size()
        uid = _uid_via_torch(rank)
    if isinstance(uid, (bytes, bytearray)):
        uid = H.UniqueId.from_bytes(bytes(uid))
    elif not isinstance(uid, H.UniqueId) and hasattr(uid, "_data"):  # the struct wrapper of the pointer-level bindings
        uid = H.UniqueId.from_bytes(uid._data.tobytes())
    if rank is None or nranks is None:
        raise NvshmemInvalid("rank and nranks are required with a unique id")
    dev = _device_ordinal(device)
    st = lib.nvshmemx_b200_init_uid(C.byref(uid), int(rank), int(nranks), int(dev))
    if st != 0:
        raise NvshmemError(f"initialisation failed with status {st}")
    _initialized = True
    atexit.register(finalize)


def finalize() -> None:
    """Frees every buffer still tracked, then shuts the library down (collective)."""
    global _initialized
    if not _initialized:
        return
    from . import memory
    memory._free_all_tracked()
    H.load().nvshmem_finalize()
    _initialized = False


def is_initialized() -> bool:
    return _initialized


def init_status() -> int:
    return int(H.load().nvshmemx_init_status())


def module_init(cumodule) -> None:
    """Fills the device-state copy of a driver-API module that was built with the device headers."""
    st = H.load().nvshmemx_cumodule_init(C.c_void_p(int(cumodule)))
    if st != 0:
        raise NvshmemError(f"nvshmemx_cumodule_init failed with status {st}")


def library_init(culibrary) -> None:
    st = H.load().nvshmemx_culibrary_init(C.c_void_p(int(culibrary)))
    if st != 0:
        raise NvshmemError(f"nvshmemx_culibrary_init failed with status {st}")
