"""Team management (reference: nvshmem4py/nvshmem/core/teams.py)."""
from __future__ import annotations

import ctypes as C
import enum

from ..bindings import host as H
from .types import NvshmemError


class Teams(enum.IntEnum):
    TEAM_INVALID = -1
    TEAM_WORLD = 0
    TEAM_SHARED = 1
    TEAM_NODE = 2
    TEAM_SAME_MYPE_NODE = 3
    TEAM_SAME_GPU = 4
    TEAM_GPU_LEADERS = 5


def get_team_unique_id() -> int:
    uid = C.c_uint64()
    H.load().nvshmemx_team_get_uniqueid(C.byref(uid))
    return int(uid.value)


def team_split_strided(parent: int, pe_start: int, pe_stride: int, pe_size: int, config: H.TeamConfig | None = None, config_mask: int = 0) -> int:
    """Collective over `parent`.  Returns the new team handle, or TEAM_INVALID on PEs that are not members."""
    new = C.c_int(-1)
    st = H.load().nvshmem_team_split_strided(int(parent), pe_start, pe_stride, pe_size, C.byref(config) if config else None, config_mask, C.byref(new))
    if st != 0:
        raise NvshmemError(f"team_split_strided failed with status {st}")
    return int(new.value)


def team_split_2d(parent: int, xrange: int, xaxis_config=None, xaxis_mask: int = 0, yaxis_config=None, yaxis_mask: int = 0) -> tuple[int, int]:
    x, y = C.c_int(-1), C.c_int(-1)
    st = H.load().nvshmem_team_split_2d(int(parent), xrange, None, 0, C.byref(x), None, 0, C.byref(y))
    if st != 0:
        raise NvshmemError(f"team_split_2d failed with status {st}")
    return int(x.value), int(y.value)


def team_init(config: H.TeamConfig, config_mask: int, npes: int, pe_idx_in_team: int) -> int:
    """Collective over the world: builds a team from arbitrary PEs that share `config.uniqueid`.
    Members pass their index and the team size; all other PEs pass ``npes=0``."""
    new = C.c_int(-1)
    st = H.load().nvshmemx_team_init(C.byref(new), C.byref(config), config_mask, npes, pe_idx_in_team)
    if st != 0:
        raise NvshmemError(f"team_init failed with status {st}")
    return int(new.value)


def team_destroy(team: int) -> None:
    H.load().nvshmem_team_destroy(int(team))


def team_translate_pe(src_team: int, src_pe: int, dest_team: int) -> int:
    return int(H.load().nvshmem_team_translate_pe(int(src_team), int(src_pe), int(dest_team)))
