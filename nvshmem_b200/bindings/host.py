"""ctypes view of ``libbshmem_host.so`` (the native host library).

Mirrors the role of nvshmem4py's generated Cython bindings
(``nvshmem4py/nvshmem/bindings/nvshmem.pyx`` in the reference): one Python
callable per C entry point, plus small POD wrappers.  The shared object is
loaded from ``nvshmem_b200/lib`` and must exist: on a GPU box a missing library
is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# BSHMEM_LIB_DIR selects another build of the native libraries (for example a sanitizer build, see utils/build.py).
LIB_DIR = Path(os.environ["BSHMEM_LIB_DIR"]) if os.environ.get("BSHMEM_LIB_DIR") else Path(__file__).resolve().parents[1] / "lib"
_lib = None

UNIQUEID_BYTES = 128

# nvshmemx_status
SUCCESS = 0
# comparison constants
CMP_EQ, CMP_NE, CMP_GT, CMP_LE, CMP_LT, CMP_GE = range(6)
SIGNAL_SET, SIGNAL_ADD = 9, 10
TEAM_INVALID, TEAM_WORLD, TEAM_SHARED, TEAM_NODE, TEAM_SAME_MYPE_NODE, TEAM_SAME_GPU, TEAM_GPU_LEADERS = -1, 0, 1, 2, 3, 4, 5
# element kinds of the collective kernels (bshmem::DType)
DT_I8, DT_U8, DT_I16, DT_U16, DT_I32, DT_U32, DT_I64, DT_U64, DT_F16, DT_BF16, DT_F32, DT_F64 = range(12)
# reduction operators (bshmem::ReduceOp)
OP_AND, OP_OR, OP_XOR, OP_MIN, OP_MAX, OP_SUM, OP_PROD = range(7)
# error bits reported by device code
ERR_WAIT_TIMEOUT, ERR_BAD_PE, ERR_BAD_ADDRESS, ERR_SCRATCH_TOO_SMALL, ERR_GLOBAL_EXIT, ERR_BAD_TEAM = 1, 2, 4, 8, 16, 32


class UniqueId(C.Structure):
    _fields_ = [("version", C.c_int), ("internal", C.c_char * 124)]

    def to_bytes(self) -> bytes:
        return bytes(C.string_at(C.addressof(self), C.sizeof(self)))

    @property
    def _data(self):
        """The 128 bytes as a writable NumPy record array over this object's memory (no copy): programs written for
        the reference package broadcast ``uid._data.view(numpy.int8)`` in place."""
        import numpy as np
        return np.frombuffer(self, dtype=np.dtype([("version", np.int32), ("internal", np.int8, (124,))], align=True), count=1).view(np.recarray)

    @property
    def ptr(self) -> int:
        return C.addressof(self)

    @classmethod
    def from_bytes(cls, raw: bytes) -> "UniqueId":
        if len(raw) != UNIQUEID_BYTES:
            raise ValueError(f"a unique id is {UNIQUEID_BYTES} bytes, got {len(raw)}")
        out = cls()
        C.memmove(C.addressof(out), raw, UNIQUEID_BYTES)
        return out


class TeamConfig(C.Structure):
    _fields_ = [("version", C.c_int), ("num_contexts", C.c_int), ("uniqueid", C.c_uint64), ("padding", C.c_char * 48)]

    def __init__(self, uniqueid: int = 0, num_contexts: int = 0):
        super().__init__()
        self.version = (2 << 16) + C.sizeof(TeamConfig)
        self.uniqueid = uniqueid
        self.num_contexts = num_contexts


class StatusBlock(C.Structure):
    _fields_ = [("error_bits", C.c_uint32), ("global_exit_req", C.c_uint32), ("global_exit_code", C.c_int32), ("timeout_count", C.c_uint32),
                ("timeout_addr", C.c_uint64), ("timeout_expected", C.c_uint64), ("timeout_found", C.c_uint64), ("timeout_where", C.c_uint32),
                ("reserved", C.c_uint32)]


def lib_path(name: str = "libbshmem_host.so") -> Path:
    return LIB_DIR / name


def load() -> C.CDLL:
    """Loads the host library once and declares the signatures used from Python."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise ImportError(f"{path} is missing: build it with `python -m nvshmem_b200.utils.build`")
    lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    vp, sz, i32, u64, stream = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64, C.c_void_p

    def sig(name, res, *args):
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = list(args)

    sig("nvshmemx_get_uniqueid", i32, C.POINTER(UniqueId))
    sig("nvshmemx_b200_init_uid", i32, C.POINTER(UniqueId), i32, i32, i32)
    sig("nvshmem_init", None)
    sig("nvshmem_finalize", None)
    sig("nvshmemx_init_status", i32)
    sig("nvshmem_my_pe", i32)
    sig("nvshmem_n_pes", i32)
    sig("nvshmem_info_get_version", None, C.POINTER(i32), C.POINTER(i32))
    sig("nvshmem_info_get_name", None, C.c_char_p)
    sig("nvshmemx_vendor_get_version_info", None, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32))
    sig("nvshmem_malloc", vp, sz)
    sig("nvshmem_calloc", vp, sz, sz)
    sig("nvshmem_align", vp, sz, sz)
    sig("nvshmem_free", None, vp)
    sig("nvshmem_ptr", vp, vp, i32)
    sig("nvshmemx_mc_ptr", vp, i32, vp)
    sig("nvshmem_team_my_pe", i32, i32)
    sig("nvshmem_team_n_pes", i32, i32)
    sig("nvshmem_team_translate_pe", i32, i32, i32, i32)
    sig("nvshmem_team_split_strided", i32, i32, i32, i32, i32, C.POINTER(TeamConfig), C.c_long, C.POINTER(i32))
    sig("nvshmem_team_split_2d", i32, i32, i32, C.POINTER(TeamConfig), C.c_long, C.POINTER(i32), C.POINTER(TeamConfig), C.c_long, C.POINTER(i32))
    sig("nvshmem_team_destroy", None, i32)
    sig("nvshmem_team_get_config", None, i32, C.POINTER(TeamConfig))
    sig("nvshmemx_team_get_uniqueid", i32, C.POINTER(u64))
    sig("nvshmemx_team_init", i32, C.POINTER(i32), C.POINTER(TeamConfig), C.c_long, i32, i32)
    sig("nvshmem_barrier_all", None)
    sig("nvshmem_barrier", i32, i32)
    sig("nvshmem_sync_all", None)
    sig("nvshmem_team_sync", i32, i32)
    sig("nvshmem_quiet", None)
    sig("nvshmem_fence", None)
    sig("nvshmemx_barrier_all_on_stream", None, stream)
    sig("nvshmemx_barrier_on_stream", i32, i32, stream)
    sig("nvshmemx_sync_all_on_stream", None, stream)
    sig("nvshmemx_team_sync_on_stream", i32, i32, stream)
    sig("nvshmemx_quiet_on_stream", None, stream)
    sig("nvshmem_putmem", None, vp, vp, sz, i32)
    sig("nvshmem_getmem", None, vp, vp, sz, i32)
    sig("nvshmem_putmem_nbi", None, vp, vp, sz, i32)
    sig("nvshmem_getmem_nbi", None, vp, vp, sz, i32)
    sig("nvshmemx_putmem_on_stream", None, vp, vp, sz, i32, stream)
    sig("nvshmemx_getmem_on_stream", None, vp, vp, sz, i32, stream)
    sig("nvshmemx_putmem_signal_on_stream", None, vp, vp, sz, vp, u64, i32, i32, stream)
    sig("nvshmemx_signal_op_on_stream", None, vp, u64, i32, i32, stream)
    sig("nvshmemx_signal_wait_until_on_stream", None, vp, i32, u64, stream)
    sig("nvshmem_signal_fetch", u64, vp)
    sig("nvshmem_long_p", None, vp, C.c_long, i32)
    sig("nvshmem_long_g", C.c_long, vp, i32)
    sig("nvshmem_long_iput", None, vp, vp, C.c_ssize_t, C.c_ssize_t, sz, i32)
    sig("nvshmem_long_atomic_fetch_add", C.c_long, vp, C.c_long, i32)
    sig("nvshmem_long_atomic_compare_swap", C.c_long, vp, C.c_long, C.c_long, i32)
    sig("nvshmem_long_atomic_swap", C.c_long, vp, C.c_long, i32)
    sig("nvshmem_long_atomic_fetch", C.c_long, vp, i32)
    sig("nvshmem_uint64_atomic_fetch_or", u64, vp, u64, i32)
    sig("nvshmemx_alltoallmem_on_stream", i32, i32, vp, vp, sz, stream)
    sig("nvshmemx_fcollectmem_on_stream", i32, i32, vp, vp, sz, stream)
    sig("nvshmemx_broadcastmem_on_stream", i32, i32, vp, vp, sz, i32, stream)
    sig("nvshmemx_b200_reduce_on_stream", i32, i32, vp, vp, sz, i32, i32, i32, stream)
    sig("nvshmemx_b200_reducescatter_on_stream", i32, i32, vp, vp, sz, i32, i32, i32, stream)
    sig("nvshmemx_b200_fcollect_on_stream", i32, i32, vp, vp, sz, i32, stream)
    sig("nvshmemx_b200_broadcast_on_stream", i32, i32, vp, vp, sz, i32, i32, stream)
    sig("nvshmemx_double2_maxloc_reduce_on_stream", i32, i32, vp, vp, sz, stream)
    sig("nvshmemx_b200_module_sync", None)
    sig("nvshmemx_b200_error_bits", C.c_uint32)
    sig("nvshmemx_b200_clear_errors", None)
    sig("nvshmemx_b200_timeout_info", C.c_uint32, C.POINTER(StatusBlock))
    sig("nvshmemx_b200_set_wait_timeout_ms", None, C.c_long)
    sig("nvshmemx_b200_topology", C.c_char_p)
    sig("nvshmemx_b200_heap_info", u64, i32)
    sig("nvshmemx_b200_release_multicast", None)
    _lib = lib
    return lib


def typed(name: str):
    """Looks up a typed entry point by its NVSHMEM name, e.g. ``nvshmemx_float_sum_reduce_on_stream``."""
    return getattr(load(), name)
