"""``nvshmem.core.nvshmem_types``: the reference package's module name for the type definitions
(nvshmem4py/nvshmem/core/nvshmem_types.py); they live in ``core.types`` and ``core.compat`` here."""
from . import (Version, NvshmemInvalid, NvshmemError, NvshmemResource, NvshmemStream, NvshmemStreamsType, MutableEnum, Teams, BufferTypes,  # noqa: F401
               NvshmemKernelObject)

__all__ = ["Version", "NvshmemInvalid", "NvshmemError", "NvshmemResource", "NvshmemStream", "NvshmemStreamsType", "MutableEnum", "Teams", "BufferTypes", "NvshmemKernelObject"]
