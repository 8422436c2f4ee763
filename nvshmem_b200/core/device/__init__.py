"""Device-side Python bindings.

The reference package offers these for Numba (nvshmem4py/nvshmem/core/device/numba: rma, amo, collective, direct),
compiled against its bitcode device library.  Numba is not part of this stack; the device-side Python path here is
Triton: :mod:`nvshmem_b200.core.device.triton` holds ``@triton.jit`` helpers (signals, fences, bounded waits,
NVLink-multicast stores and in-switch reductions) that user kernels call on peer and multicast views of symmetric
tensors (``get_peer_tensor`` / ``get_multicast_tensor``).  ``nvshmem_b200.core.device.numba`` does not exist and
importing it says so.
"""


def __getattr__(name: str):
    if name == "numba":
        raise ImportError("the Numba device bindings of the reference package are not offered; use nvshmem.core.device.triton "
                          "(Triton helpers on peer / multicast views of symmetric tensors) or the C++ device headers")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
