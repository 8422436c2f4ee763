"""nvshmem4py-compatible Python layer (``nvshmem.core`` in the reference).

Same call names and argument order as ``nvshmem4py/nvshmem/core``: ``init``,
``finalize``, ``get_unique_id``, ``my_pe``, ``n_pes``, ``tensor`` /
``free_tensor`` / ``get_peer_tensor`` / ``get_multicast_tensor``, the on-stream
RMA calls (``put``, ``get``, ``put_signal``, ``signal_op``, ``signal_wait``,
``quiet``), the collectives (``reduce``, ``reducescatter``, ``alltoall``,
``fcollect``, ``broadcast``, ``barrier``, ``sync``) and the team calls.
"""
from .init_fini import (finalize, get_unique_id, get_version, init, init_status, is_initialized,  # noqa: F401
                        library_init, module_init)
from .direct import my_pe, n_pes, team_my_pe, team_n_pes, error_bits, clear_errors, set_wait_timeout_ms, set_ce_collectives, topology, heap_info  # noqa: F401
from .memory import (Buffer, buffer, free, get_peer_buffer, get_multicast_buffer, register_external_buffer, unregister_external_buffer,  # noqa: F401
                     tensor, bytetensor, free_tensor, get_peer_tensor, get_multicast_tensor, register_external_tensor,
                     tensor_ptr, peer_ptr)
from .rma import put, get, put_signal, signal_op, signal_wait, signal_fetch, quiet  # noqa: F401
from .collective import (reduce, reducescatter, alltoall, fcollect, broadcast, barrier, barrier_all, sync, sync_all,  # noqa: F401
                         collective_on_buffer, maxloc)
from .teams import (Teams, team_split_strided, team_split_2d, team_destroy, team_init, team_translate_pe, get_team_unique_id)  # noqa: F401
from .types import ComparisonType, SignalOp, NvshmemError, NvshmemInvalid, NvshmemStream  # noqa: F401
from .compat import (UniqueID, TeamConfig, TeamUniqueId, BufferTypes, InitStatus, NvshmemStreamsType, NvshmemWarning, MutableEnum, Version,  # noqa: F401
                     NvshmemKernelObject, NvshmemResource, module_finalize, library_finalize, dtype_nbytes, get_size, tensor_get_buffer,
                     unregister_external_tensor, array, bytearray, array_get_buffer, free_array, get_peer_array, get_multicast_array,
                     register_external_array, unregister_external_array)
