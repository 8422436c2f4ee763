"""Flat, pointer-level bindings: one Python function per C entry point, addresses passed as plain integers.

This is the layer that the reference's Python package exposes as ``nvshmem.bindings`` (generated Cython there:
nvshmem4py/nvshmem/bindings/nvshmem.pyx; the same function names, argument orders and enum names here), for code that
manages its own memory and streams: ``malloc`` returns an ``int``, ``float_sum_reduce_on_stream(team, dest, src, n,
stream)`` takes integers, structures (``UniqueId``, ``InitAttr``, ``TeamConfig``, ``TeamUniqueId``) are NumPy-backed
arrays of C structs whose ``.ptr`` is the address to pass.  A non-zero status from the library raises
:class:`NVSHMEMError`.  The higher layer (``nvshmem.core``) does not go through this module; both sit on the same
shared library.
"""
from __future__ import annotations

import ctypes as _C
from enum import IntEnum as _IntEnum

import numpy as _np

from . import host as _H

_raw = None


def _lib() -> _C.CDLL:
    """A handle of its own on the host library: every pointer is declared ``void*`` here, whatever the typed
    declarations of the other layer say."""
    global _raw
    if _raw is None:
        _H.load()
        _raw = _C.CDLL(str(_H.lib_path()), mode=_C.RTLD_GLOBAL)
    return _raw


# ---------------------------------------------------------------------------------------------- structures
class _StructArray:
    """``size`` C structs in one NumPy record array.  Fields read as scalars when there is one struct."""

    _dtype: _np.dtype = None

    def __init__(self, size: int = 1):
        self._data = _np.zeros(size, dtype=self._dtype).view(_np.recarray)
        self._defaults()

    def _defaults(self) -> None:
        pass

    def __repr__(self):
        kind = type(self).__name__
        return f"<{__name__}.{kind}{'' if self._data.size == 1 else f'_Array_{self._data.size}'} object at {hex(id(self))}>"

    @property
    def ptr(self) -> int:
        return self._data.ctypes.data

    def __int__(self):
        if self._data.size != 1:
            raise TypeError("int() needs a single struct; use .ptr for the address of an array")
        return self._data.ctypes.data

    def __len__(self):
        return self._data.size

    def __eq__(self, other):
        return isinstance(other, _StructArray) and self._data.dtype == other._data.dtype and self._data.size == other._data.size and \
            self._data.tobytes() == other._data.tobytes()

    def __hash__(self):
        return id(self)

    def __getitem__(self, key):
        if isinstance(key, int):
            n = self._data.size
            if not -n <= key < n:
                raise IndexError("index is out of bounds")
            key %= n
            return type(self).from_data(self._data[key:key + 1])
        out = self._data[key]
        return type(self).from_data(out) if isinstance(out, _np.ndarray) and out.dtype == self._dtype else out

    def __setitem__(self, key, val):
        self._data[key] = val._data if isinstance(val, _StructArray) else val

    @classmethod
    def from_data(cls, data):
        """Wraps an existing NumPy array of this struct type (no copy)."""
        if not isinstance(data, _np.ndarray) or data.dtype != cls._dtype or data.ndim != 1:
            raise ValueError(f"data must be a one-dimensional NumPy array of dtype {cls._dtype}")
        obj = cls.__new__(cls)
        obj._data = data.view(_np.recarray)
        return obj

    @classmethod
    def from_ptr(cls, ptr: int, size: int = 1, readonly: bool = False):
        """Wraps ``size`` structs at address ``ptr`` (the memory stays the caller's)."""
        if ptr == 0:
            raise ValueError("ptr must not be null")
        buf = (_C.c_char * (cls._dtype.itemsize * size)).from_address(ptr)
        arr = _np.frombuffer(buf, dtype=cls._dtype, count=size)
        if readonly:
            arr.flags.writeable = False
        return cls.from_data(arr)


def _field(name):
    def get(self):
        col = self._data[name]
        return col[0].item() if self._data.size == 1 and col.ndim == 1 else col

    def put(self, val):
        self._data[name] = val
    return property(get, put)


def _struct(name, fields, defaults=None, doc=""):
    dt = _np.dtype(fields, align=True)
    ns = {"_dtype": dt, "__doc__": doc}
    for f in dt.names:
        ns[f] = _field(f)
    if defaults:
        def _defaults(self, _d=defaults):
            for k, v in _d.items():
                self._data[k] = v(dt) if callable(v) else v
        ns["_defaults"] = _defaults
    return type(name, (_StructArray,), ns)


uniqueid_dtype = _np.dtype([("version", _np.int32), ("internal", _np.int8, (124,))], align=True)
uniqueid = _struct("uniqueid", [("version", _np.int32), ("internal", _np.int8, (124,))],
                   {"version": lambda dt: (1 << 16) + dt.itemsize}, "nvshmemx_uniqueid_t: 128 bytes that name a job's bootstrap root.")
team_uniqueid_dtype = _np.dtype([("value", _np.uint64)], align=True)
team_uniqueid = _struct("team_uniqueid", [("value", _np.uint64)], None, "nvshmemx_team_uniqueid_t: a 64-bit team identifier.")
# args: the nvshmemx_init_args_t block, opaque at this level (set_attr_uniqueid_args fills it)
init_attr_dtype = _np.dtype([("version", _np.int32), ("mpi_comm", _np.intp), ("args", _np.int8, (128,))], align=True)
InitAttr = _struct("InitAttr", [("version", _np.int32), ("mpi_comm", _np.intp), ("args", _np.int8, (128,))],
                   {"version": lambda dt: (2 << 16) + dt.itemsize}, "nvshmemx_init_attr_t.")
team_config_dtype = _np.dtype([("version", _np.int32), ("num_contexts", _np.int32), ("uniqueid", _np.uint64), ("padding", _np.int8, (48,))], align=True)
TeamConfig = _struct("TeamConfig", [("version", _np.int32), ("num_contexts", _np.int32), ("uniqueid", _np.uint64), ("padding", _np.int8, (48,))],
                     {"version": lambda dt: (2 << 16) + dt.itemsize}, "nvshmem_team_config_t.")


class UniqueId(uniqueid):
    pass


class TeamUniqueId(team_uniqueid):
    pass


assert uniqueid._dtype.itemsize == 128 and InitAttr._dtype.itemsize == 144 and TeamConfig._dtype.itemsize == 64


def _init_args_defaults(self):
    # NVSHMEMX_INIT_ARGS_INITIALIZER inside the attribute block: version, uid_args {version, id, myrank, nranks}, cuda_device_id
    raw = self._data["args"]
    for i in range(self._data.size):
        view = raw[i].view(_np.int32)
        view[0] = (2 << 16) + 128
        view[2] = (1 << 16) + 24          # uid_args.version (after 4 bytes of padding: the struct holds a pointer)
        view[6], view[7] = -1, -1         # myrank, nranks
        view[8] = -1                      # cuda_device_id


_base_defaults = InitAttr._defaults


def _init_attr_defaults(self):
    _base_defaults(self)
    _init_args_defaults(self)


InitAttr._defaults = _init_attr_defaults


# ---------------------------------------------------------------------------------------------- enums
class Signal_op(_IntEnum):
    SIGNAL_SET = 9
    SIGNAL_ADD = 10


class Cmp_type(_IntEnum):
    CMP_EQ = 0
    CMP_NE = 1
    CMP_GT = 2
    CMP_LE = 3
    CMP_LT = 4
    CMP_GE = 5
    CMP_SENTINEL = 0x7fffffff


class Thread_support(_IntEnum):
    THREAD_SINGLE = 0
    THREAD_FUNNELED = 1
    THREAD_SERIALIZED = 2
    THREAD_MULTIPLE = 3
    THREAD_TYPE_SENTINEL = 0x7fffffff


class Proxy_status(_IntEnum):
    _PROXY_GLOBAL_EXIT_NOT_REQUESTED = 0
    _PROXY_GLOBAL_EXIT_INIT = 1
    _PROXY_GLOBAL_EXIT_REQUESTED = 2
    _PROXY_GLOBAL_EXIT_FINISHED = 3
    _PROXY_GLOBAL_EXIT_MAX_STATE = 0x7fffffff


class Init_status(_IntEnum):
    STATUS_NOT_INITIALIZED = 0
    STATUS_IS_BOOTSTRAPPED = 1
    STATUS_IS_INITIALIZED = 2
    STATUS_LIMITED_MPG = 3
    STATUS_FULL_MPG = 4
    STATUS_INVALID = 0x7fffffff


class Qp_handle_index(_IntEnum):
    QP_HOST = 0
    QP_DEFAULT = 1
    QP_ANY = 0x7fffffff
    QP_ALL = 0x7fffffff


class Pe_index(_IntEnum):
    PE_INVALID = -1
    PE_ANY = -1
    PE_ALL = 1 << 15


class Team_id(_IntEnum):
    # In this library a predefined team's handle is its index in the team pool.
    TEAM_INVALID = -1
    TEAM_WORLD = 0
    TEAM_WORLD_INDEX = 0
    TEAM_SHARED = 1
    TEAM_SHARED_INDEX = 1
    TEAM_NODE = 2
    TEAM_NODE_INDEX = 2
    TEAM_SAME_MYPE_NODE = 3
    TEAM_SAME_MYPE_NODE_INDEX = 3
    TEAM_SAME_GPU = 4
    TEAM_SAME_GPU_INDEX = 4
    TEAM_GPU_LEADERS = 5
    TEAM_GPU_LEADERS_INDEX = 5
    TEAMS_MIN = 6
    TEAM_INDEX_MAX = 0x7fff


class Status(_IntEnum):
    SUCCESS = 0
    ERROR_INVALID_VALUE = 1
    ERROR_OUT_OF_MEMORY = 2
    ERROR_NOT_SUPPORTED = 3
    ERROR_SYMMETRY = 4
    ERROR_GPU_NOT_SELECTED = 5
    ERROR_COLLECTIVE_LAUNCH_FAILED = 6
    ERROR_INTERNAL = 7
    ERROR_SENTINEL = 0x7fffffff


class Flags(_IntEnum):
    INIT_THREAD_PES = 1
    INIT_WITH_MPI_COMM = 1 << 1
    INIT_WITH_SHMEM = 1 << 2
    INIT_WITH_UNIQUEID = 1 << 3
    INIT_MAX = 1 << 31


class NVSHMEMError(Exception):
    def __init__(self, status):
        self.status = status
        super().__init__(f"Status code {status}")

    def __reduce__(self):
        return (type(self), (self.status,))


def check_status(status: int) -> None:
    if status != 0:
        raise NVSHMEMError(status)


# ---------------------------------------------------------------------------------------------- functions
_P, _SZ, _I, _U64, _L = _C.c_void_p, _C.c_size_t, _C.c_int, _C.c_uint64, _C.c_long
_declared: dict = {}


def _fn(symbol, res, *args):
    f = _declared.get(symbol)
    if f is None:
        f = getattr(_lib(), symbol)
        f.restype = res
        f.argtypes = list(args)
        _declared[symbol] = f
    return f


def _addr(v) -> int:
    """Accepts an int or anything with ``.ptr`` / ``__int__`` (the struct wrappers above)."""
    return int(v.ptr) if hasattr(v, "ptr") else int(v)


def init_status() -> int:
    return _fn("nvshmemx_init_status", _I)()


def my_pe() -> int:
    return _fn("nvshmem_my_pe", _I)()


def n_pes() -> int:
    return _fn("nvshmem_n_pes", _I)()


def info_get_version(major, minor) -> None:
    """Writes two C ints at the given addresses."""
    _fn("nvshmem_info_get_version", None, _P, _P)(_addr(major), _addr(minor))


def vendor_get_version_info(major, minor, patch) -> None:
    _fn("nvshmemx_vendor_get_version_info", None, _P, _P, _P)(_addr(major), _addr(minor), _addr(patch))


def malloc(size: int) -> int:
    return _fn("nvshmem_malloc", _P, _SZ)(size) or 0


def calloc(count: int, size: int) -> int:
    return _fn("nvshmem_calloc", _P, _SZ, _SZ)(count, size) or 0


def align(alignment: int, size: int) -> int:
    return _fn("nvshmem_align", _P, _SZ, _SZ)(alignment, size) or 0


def free(ptr) -> None:
    _fn("nvshmem_free", None, _P)(_addr(ptr))


def ptr(dest, pe: int) -> int:
    return _fn("nvshmem_ptr", _P, _P, _I)(_addr(dest), pe) or 0


def mc_ptr(team: int, ptr) -> int:  # noqa: A002 - the reference's parameter name
    return _fn("nvshmemx_mc_ptr", _P, _I, _P)(team, _addr(ptr)) or 0


def barrier(team: int) -> None:
    check_status(_fn("nvshmem_barrier", _I, _I)(team))


def barrier_all() -> None:
    _fn("nvshmem_barrier_all", None)()


def team_my_pe(team: int) -> int:
    return _fn("nvshmem_team_my_pe", _I, _I)(team)


def team_n_pes(team: int) -> int:
    return _fn("nvshmem_team_n_pes", _I, _I)(team)


def team_get_config(team: int, config) -> None:
    _fn("nvshmem_team_get_config", None, _I, _P)(team, _addr(config))


def team_translate_pe(src_team: int, src_pe: int, dest_team: int) -> int:
    return _fn("nvshmem_team_translate_pe", _I, _I, _I, _I)(src_team, src_pe, dest_team)


def team_split_strided(parent_team: int, pe_start: int, pe_stride: int, pe_size: int, config, config_mask: int, new_team) -> None:
    """``new_team`` is the address of a C int that receives the handle."""
    check_status(_fn("nvshmem_team_split_strided", _I, _I, _I, _I, _I, _P, _L, _P)(parent_team, pe_start, pe_stride, pe_size, _addr(config), config_mask,
                                                                                 _addr(new_team)))


def team_split_2d(parent_team: int, xrange: int, xaxis_config, xaxis_mask: int, xaxis_team, yaxis_config, yaxis_mask: int, yaxis_team) -> None:
    check_status(_fn("nvshmem_team_split_2d", _I, _I, _I, _P, _L, _P, _P, _L, _P)(parent_team, xrange, _addr(xaxis_config), xaxis_mask, _addr(xaxis_team),
                                                                                _addr(yaxis_config), yaxis_mask, _addr(yaxis_team)))


def team_get_uniqueid(uniqueid) -> None:  # noqa: A002
    check_status(_fn("nvshmemx_team_get_uniqueid", _I, _P)(_addr(uniqueid)))


def team_init(team, config, config_mask: int, npes: int, pe_idx_in_team: int) -> None:
    check_status(_fn("nvshmemx_team_init", _I, _P, _P, _L, _I, _I)(_addr(team), _addr(config), config_mask, npes, pe_idx_in_team))


def team_destroy(team: int) -> None:
    _fn("nvshmem_team_destroy", None, _I)(team)


def barrier_on_stream(team: int, stream: int) -> None:
    check_status(_fn("nvshmemx_barrier_on_stream", _I, _I, _P)(team, stream))


def barrier_all_on_stream(stream: int) -> None:
    _fn("nvshmemx_barrier_all_on_stream", None, _P)(stream)


def team_sync_on_stream(team: int, stream: int) -> int:
    return _fn("nvshmemx_team_sync_on_stream", _I, _I, _P)(team, stream)


def sync_all_on_stream(stream: int) -> None:
    _fn("nvshmemx_sync_all_on_stream", None, _P)(stream)


def hostlib_init_attr(flags: int, attr) -> None:
    check_status(_fn("nvshmemx_hostlib_init_attr", _I, _C.c_uint, _P)(flags, _addr(attr)))


def hostlib_finalize() -> None:
    _fn("nvshmemx_hostlib_finalize", None)()


def set_attr_uniqueid_args(myrank: int, nranks: int, uniqueid, attr) -> None:  # noqa: A002
    check_status(_fn("nvshmemx_set_attr_uniqueid_args", _I, _I, _I, _P, _P)(myrank, nranks, _addr(uniqueid), _addr(attr)))


def set_attr_mpi_comm_args(mpi_comm, nvshmem_attr) -> None:
    check_status(_fn("nvshmemx_set_attr_mpi_comm_args", _I, _P, _P)(_addr(mpi_comm), _addr(nvshmem_attr)))


def get_uniqueid(uniqueid) -> None:  # noqa: A002
    check_status(_fn("nvshmemx_get_uniqueid", _I, _P)(_addr(uniqueid)))


def cumodule_init(module: int) -> int:
    return _fn("nvshmemx_cumodule_init", _I, _P)(module)


def cumodule_finalize(module: int) -> int:
    return _fn("nvshmemx_cumodule_finalize", _I, _P)(module)


def culibrary_init(library: int) -> int:
    return _fn("nvshmemx_culibrary_init", _I, _P)(library)


def culibrary_finalize(library: int) -> int:
    return _fn("nvshmemx_culibrary_finalize", _I, _P)(library)


def buffer_register_symmetric(buf_ptr, size: int, flags: int) -> int:
    return _fn("nvshmemx_buffer_register_symmetric", _P, _P, _SZ, _I)(_addr(buf_ptr), size, flags) or 0


def buffer_unregister_symmetric(mmap_ptr, size: int) -> int:
    return _fn("nvshmemx_buffer_unregister_symmetric", _I, _P, _SZ)(_addr(mmap_ptr), size)


def putmem_on_stream(dest, source, bytes: int, pe: int, cstrm: int) -> None:  # noqa: A002
    _fn("nvshmemx_putmem_on_stream", None, _P, _P, _SZ, _I, _P)(_addr(dest), _addr(source), bytes, pe, cstrm)


def getmem_on_stream(dest, source, bytes: int, pe: int, cstrm: int) -> None:  # noqa: A002
    _fn("nvshmemx_getmem_on_stream", None, _P, _P, _SZ, _I, _P)(_addr(dest), _addr(source), bytes, pe, cstrm)


def putmem_signal_on_stream(dest, source, bytes: int, sig_addr, signal: int, sig_op: int, pe: int, cstrm: int) -> None:  # noqa: A002
    _fn("nvshmemx_putmem_signal_on_stream", None, _P, _P, _SZ, _P, _U64, _I, _I, _P)(_addr(dest), _addr(source), bytes, _addr(sig_addr), signal, sig_op, pe, cstrm)


def quiet_on_stream(cstrm: int) -> None:
    _fn("nvshmemx_quiet_on_stream", None, _P)(cstrm)


def signal_op_on_stream(sig_addr, signal: int, sig_op: int, pe: int, cstrm: int) -> None:
    _fn("nvshmemx_signal_op_on_stream", None, _P, _U64, _I, _I, _P)(_addr(sig_addr), signal, sig_op, pe, cstrm)


def signal_wait_until_on_stream(sig_addr, cmp: int, cmp_value: int, cstream: int) -> None:
    _fn("nvshmemx_signal_wait_until_on_stream", None, _P, _I, _U64, _P)(_addr(sig_addr), cmp, cmp_value, cstream)


# ---------------------------------------------------------------------------------------------- typed collectives
# <type>_{alltoall,broadcast,fcollect}_on_stream and <type>_{op}_{reduce,reducescatter}_on_stream for every element type
# name and operator the library exports (counts are in elements).  Defined on first use of the module's attribute.
TYPE_NAMES = ("int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64", "size", "char", "schar", "short", "int", "long", "longlong", "uchar", "ushort",
              "uint", "ulong", "ulonglong", "ptrdiff", "half", "bfloat16", "float", "double")
REDUCE_OPS = ("and", "or", "xor", "min", "max", "sum", "prod")


def _make_collective(name: str):
    symbol = "nvshmemx_" + name
    if not hasattr(_lib(), symbol):
        return None
    if name.endswith("_broadcast_on_stream"):
        def call(team: int, dest, src, nelem: int, pe_root: int, stream: int) -> None:
            check_status(_fn(symbol, _I, _I, _P, _P, _SZ, _I, _P)(team, _addr(dest), _addr(src), nelem, pe_root, stream))
    else:
        def call(team: int, dest, src, nelem: int, stream: int) -> None:
            check_status(_fn(symbol, _I, _I, _P, _P, _SZ, _P)(team, _addr(dest), _addr(src), nelem, stream))
    call.__name__ = call.__qualname__ = name
    call.__doc__ = f"{symbol}: addresses as integers, the count in elements."
    return call


def _collective_names():
    for t in TYPE_NAMES:
        for kind in ("alltoall", "broadcast", "fcollect"):
            yield f"{t}_{kind}_on_stream"
        for op in REDUCE_OPS:
            yield f"{t}_{op}_reduce_on_stream"
            yield f"{t}_{op}_reducescatter_on_stream"


_COLLECTIVES = frozenset(_collective_names())


def __getattr__(name: str):
    if name in _COLLECTIVES:
        fn = _make_collective(name)
        if fn is not None:
            globals()[name] = fn
            return fn
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | _COLLECTIVES)
