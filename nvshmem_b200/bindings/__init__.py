"""Bindings of the native host library.

* ``host``     – the ctypes loader with typed declarations that the Python layer (``nvshmem_b200.core``) uses.
* ``nvshmem``  – the flat, pointer-level API with the reference package's names (``nvshmem.bindings`` there): every
  public name of that module is also reachable from this package, e.g. ``bindings.malloc``,
  ``bindings.float_sum_reduce_on_stream``, ``bindings.Team_id``.
"""
from . import host  # noqa: F401
from . import nvshmem  # noqa: F401
from .nvshmem import *  # noqa: F401,F403


def __getattr__(name: str):
    # the typed collectives of the flat module are defined on first use
    if not name.startswith("_"):
        return getattr(nvshmem, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | set(dir(nvshmem)))
