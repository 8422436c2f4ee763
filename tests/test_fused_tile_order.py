"""Invariants of the fused GEMM's tile order, checked on the CPU through a host hook of the fused library:
what the kernel's flag indexing and the CTA-pair variant rely on.  No GPU."""
import ctypes as C
import itertools

import pytest

PLAIN, RS, AR, AG = 0, 1, 2, 3
BM, BN = 128, 256


def _lib():
    from nvshmem_b200.bindings import host as H
    path = H.lib_path("libbshmem_fused.so")
    if not path.exists():
        from nvshmem_b200.utils.build import build_all
        build_all(only="fused")
    lib = C.CDLL(str(path))
    lib.bshmem_fused_test_tile_info.argtypes = [C.c_int] * 6 + [C.POINTER(C.c_int)]
    return lib


def _order(lib, mode, M, N, rank, npes):
    total = (M // BM) * (N // BN)
    out = (C.c_int * 5)()
    tiles = []
    for t in range(total):
        assert lib.bshmem_fused_test_tile_info(mode, M, N, rank, npes, t, out) == 0
        tiles.append(tuple(out))
    assert lib.bshmem_fused_test_tile_info(mode, M, N, rank, npes, total, out) != 0  # out of range is refused
    return tiles


@pytest.mark.parametrize("mode,npes,M,N", [(PLAIN, 1, 1024, 512), (RS, 2, 1024, 768), (RS, 8, 8192, 1024), (AR, 4, 2048, 512), (AG, 8, 4096, 768), (AG, 3, 768, 256)])
def test_every_tile_once_and_blocks_in_the_documented_order(mode, npes, M, N):
    lib = _lib()
    tmr, tiles_n = M // npes // BM, N // BN
    for rank in range(npes):
        tiles = _order(lib, mode, M, N, rank, npes)
        # every output tile exactly once
        assert sorted((m, n) for m, n, *_ in tiles) == sorted(itertools.product(range(M // BM), range(tiles_n)))
        for m_tile, n_tile, peer, m_local, idx in tiles:
            assert m_tile == peer * tmr + m_local and 0 <= m_local < tmr       # the tile lies in `peer`'s block of rows
            assert idx == n_tile * tmr + m_local                               # flag index inside the block: m fastest
        peers_in_order = [p for p, _ in itertools.groupby(t[2] for t in tiles)]
        assert len(peers_in_order) == npes and sorted(peers_in_order) == list(range(npes))   # one contiguous run per block
        if mode in (RS, AR):
            assert peers_in_order == [(rank + 1 + o) % npes for o in range(npes)]             # nearest first, own rows last
        if mode == AG:
            assert peers_in_order == [(rank - o) % npes for o in range(npes)]                 # own shard first
        # flag indices are unique inside a block (one flag per tile and sender)
        for p in range(npes):
            idxs = [t[4] for t in tiles if t[2] == p]
            assert sorted(idxs) == list(range(tmr * tiles_n))


@pytest.mark.parametrize("mode,npes,M,N", [(PLAIN, 1, 1024, 512), (RS, 8, 8192, 512), (AR, 2, 1024, 256), (AG, 4, 2048, 768)])
def test_cta_pairs_get_two_row_tiles_of_one_column_block(mode, npes, M, N):
    """With an even number of 128-row tiles per PE, positions 2u and 2u+1 of the order share their 256 columns and
    their owner and are adjacent in m: what lets two CTAs share one B tile."""
    lib = _lib()
    assert (M // npes // BM) % 2 == 0
    for rank in range(npes):
        tiles = _order(lib, mode, M, N, rank, npes)
        assert len(tiles) % 2 == 0
        for u in range(0, len(tiles), 2):
            a, b = tiles[u], tiles[u + 1]
            assert a[1] == b[1] and a[2] == b[2] and b[0] == a[0] + 1 and a[3] % 2 == 0, (rank, u, a, b)


def test_all_gather_units_tile_a_block_and_are_dealt_to_every_cta():
    """The all-gather mode cuts each 128-row block into units and deals them round-robin to the CTAs; the arrival
    counter of a block must grow by exactly `units_per_block`, units must be whole 16-byte pieces that tile the block,
    and a row is only split while there are more CTAs than units."""
    lib = _lib()
    lib.bshmem_fused_test_ag_units.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_int)]
    out = (C.c_int * 2)()
    for K in (64, 128, 1024, 2048, 3584, 8192, 28672):
        for grid in (1, 2, 3, 64, 128, 132, 148, 296):
            assert lib.bshmem_fused_test_ag_units(K, grid, out) == 0
            unit, per_block = out[0], out[1]
            assert unit % 16 == 0 and unit * per_block == BM * K * 2
            assert per_block >= BM and (per_block == BM or unit >= 2048)
            assert per_block >= grid or unit < 4096       # every CTA gets a unit of each block unless units are small already
            delivered = sum(len(range(b, per_block, grid)) for b in range(grid))
            assert delivered == per_block
    assert lib.bshmem_fused_test_ag_units(100, 148, out) != 0
    assert lib.bshmem_fused_test_ag_units(8192, 148, out) == 0 and (out[0], out[1]) == (8192, 256)


@pytest.mark.parametrize("mode,npes,M,N", [(RS, 2, 1024, 768), (RS, 8, 8192, 1024), (AR, 4, 2048, 512), (RS, 3, 768, 256)])
def test_switch_path_walks_the_output_in_one_order_on_every_pe(mode, npes, M, N):
    """Switch path of RS / AR: the order does not depend on the rank, m runs fastest over ALL rows (so the owner changes
    every M/npes rows and every wave of CTAs holds tiles of every owner), and the flag index is the position of the
    tile among its owner's tiles in that same order (what the reducing warps count through)."""
    lib = _lib()
    SW = 0x100
    tmr, tiles_n, tiles_m = M // npes // BM, N // BN, M // BM
    orders = [_order(lib, mode | SW, M, N, rank, npes) for rank in range(npes)]
    assert all(o == orders[0] for o in orders)
    tiles = orders[0]
    assert [(m, n) for m, n, *_ in tiles] == [(t % tiles_m, t // tiles_m) for t in range(len(tiles))]
    for owner in range(npes):
        mine = [t for t in tiles if t[2] == owner]
        assert [t[4] for t in mine] == list(range(tmr * tiles_n))
        assert all(m == owner * tmr + ml for m, _, _, ml, _ in mine)
    if tmr % 2 == 0:
        for u in range(0, len(tiles), 2):
            a, b = tiles[u], tiles[u + 1]
            assert a[1] == b[1] and a[2] == b[2] and b[0] == a[0] + 1
