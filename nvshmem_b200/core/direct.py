"""Direct queries (reference: nvshmem4py/nvshmem/core/direct.py) and this library's status extensions."""
from __future__ import annotations

import ctypes as C

from ..bindings import host as H


def my_pe() -> int:
    return int(H.load().nvshmem_my_pe())


def n_pes() -> int:
    return int(H.load().nvshmem_n_pes())


def team_my_pe(team: int) -> int:
    return int(H.load().nvshmem_team_my_pe(int(team)))


def team_n_pes(team: int) -> int:
    return int(H.load().nvshmem_team_n_pes(int(team)))


def error_bits() -> int:
    """Error bits set by device code since the last clear (``H.ERR_*``); bounded waits report here."""
    return int(H.load().nvshmemx_b200_error_bits())


def clear_errors() -> None:
    H.load().nvshmemx_b200_clear_errors()


def timeout_info() -> dict:
    blk = H.StatusBlock()
    n = H.load().nvshmemx_b200_timeout_info(C.byref(blk))
    return {"count": int(n), "addr": int(blk.timeout_addr), "expected": int(blk.timeout_expected), "found": int(blk.timeout_found), "where": int(blk.timeout_where)}


def set_wait_timeout_ms(ms: int) -> None:
    H.load().nvshmemx_b200_set_wait_timeout_ms(int(ms))


def set_ce_collectives(min_bytes: int) -> None:
    """On-stream alltoall / fcollect / broadcast of at least `min_bytes` use the copy engines (0: never, the default).
    Every PE must set the same value."""
    lib = H.load()
    lib.nvshmemx_b200_set_ce_collectives.restype = None
    lib.nvshmemx_b200_set_ce_collectives.argtypes = [C.c_size_t]
    lib.nvshmemx_b200_set_ce_collectives(int(min_bytes))


def topology() -> str:
    return H.load().nvshmemx_b200_topology().decode()


def heap_info() -> dict:
    lib = H.load()
    keys = ["base", "stride", "backed", "mc_base", "chunks", "in_use", "digest"]
    return {k: int(lib.nvshmemx_b200_heap_info(i)) for i, k in enumerate(keys)}
