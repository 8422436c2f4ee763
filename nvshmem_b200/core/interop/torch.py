"""``nvshmem.core.interop.torch``: symmetric torch tensors (reference: nvshmem4py/nvshmem/core/interop/torch.py)."""
from .. import (bytetensor, tensor, free_tensor, tensor_get_buffer, get_peer_tensor, get_multicast_tensor,  # noqa: F401
                register_external_tensor, unregister_external_tensor)

__all__ = ["bytetensor", "tensor", "free_tensor", "tensor_get_buffer", "get_peer_tensor", "get_multicast_tensor", "register_external_tensor", "unregister_external_tensor"]
