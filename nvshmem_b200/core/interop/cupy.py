"""``nvshmem.core.interop.cupy``: symmetric CuPy arrays (reference: nvshmem4py/nvshmem/core/interop/cupy.py).  The
functions raise a clear error while CuPy is not installed."""
from .. import (bytearray, array, free_array, array_get_buffer, get_peer_array, get_multicast_array, register_external_array,  # noqa: F401,A004
                unregister_external_array)

__all__ = ["bytearray", "array", "free_array", "array_get_buffer", "get_peer_array", "get_multicast_array", "register_external_array", "unregister_external_array"]
