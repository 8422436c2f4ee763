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
