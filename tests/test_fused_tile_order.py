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


def test_all_gather_sender_plan_invariants():
    """The split of a PE's shard over the sender CTAs: units cover the shard exactly, nest with the 128-row blocks
    (arrival counters are per block), are copied in power-of-two pieces, and come in even numbers for CTA pairs."""
    lib = _lib()
    lib.bshmem_fused_test_ag_plan.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_longlong)]
    out = (C.c_longlong * 6)()
    checked = 0
    for npes in (2, 3, 4, 8):
        for tmr in (1, 2, 3, 4, 6, 8, 16):
            for K in (64, 192, 1024, 8192):
                for req in (0, 1, 2, 3, 5, 8, 16, 24, 32):
                    for pair in (0, 1):
                        M = npes * tmr * BM
                        assert lib.bshmem_fused_test_ag_plan(M, K, npes, req, pair, out) == 0, (npes, tmr, K, req, pair)
                        n_comm, is_pair, unit, piece, parts, per_unit = [int(v) for v in out]
                        rows = tmr * BM
                        shard = rows * K * 2
                        assert 1 <= n_comm <= (req or 16) and n_comm * unit == shard
                        assert piece & (piece - 1) == 0 and 16 <= piece <= 16384 and unit % piece == 0
                        if n_comm >= tmr:
                            assert n_comm % tmr == 0 and parts == n_comm // tmr and per_unit == 1
                            assert rows % n_comm == 0 and BM % (rows // n_comm) == 0      # a unit is a whole fraction of one block
                        else:
                            assert tmr % n_comm == 0 and parts == 1 and per_unit == tmr // n_comm
                        if is_pair:
                            assert pair and tmr % 2 == 0 and n_comm % 2 == 0
                        checked += 1
    assert checked > 1000
    # the benchmark's all-gather shape: 16 senders, half a block each, 16 KB pieces
    assert lib.bshmem_fused_test_ag_plan(8192, 8192, 8, 0, 1, out) == 0
    assert [int(v) for v in out] == [16, 1, 1 << 20, 16384, 2, 1]
