"""Property tests of the symmetric-heap allocator through its C test hooks (no GPU): random sequences of
allocate / free / grow never hand out overlapping or misaligned ranges, keep the free list consistent, return
every byte when everything is freed, and two allocators fed the same sequence agree (the symmetry every PE relies on)."""
import ctypes as C

from hypothesis import given, settings, strategies as st

from nvshmem_b200.bindings import host as H


def _lib():
    lib = H.load()
    lib.bshmem_test_alloc_new.restype = C.c_void_p
    lib.bshmem_test_alloc_new.argtypes = [C.c_ulonglong]
    lib.bshmem_test_alloc_delete.argtypes = [C.c_void_p]
    lib.bshmem_test_alloc_grow.argtypes = [C.c_void_p, C.c_ulonglong, C.c_ulonglong]
    lib.bshmem_test_alloc_malloc.restype = C.c_longlong
    lib.bshmem_test_alloc_malloc.argtypes = [C.c_void_p, C.c_ulonglong, C.c_ulonglong]
    lib.bshmem_test_alloc_free.argtypes = [C.c_void_p, C.c_ulonglong]
    lib.bshmem_test_alloc_check.argtypes = [C.c_void_p]
    for name in ("bshmem_test_alloc_digest", "bshmem_test_alloc_in_use", "bshmem_test_alloc_largest_free"):
        getattr(lib, name).restype = C.c_ulonglong
        getattr(lib, name).argtypes = [C.c_void_p]
    return lib


ops = st.lists(st.one_of(st.tuples(st.just("alloc"), st.integers(1, 1 << 20), st.sampled_from([0, 64, 512, 4096, 65536])),
                         st.tuples(st.just("free"), st.integers(0, 1 << 30), st.just(0)),
                         st.tuples(st.just("grow"), st.integers(1, 8), st.just(0))), min_size=1, max_size=120)


@settings(max_examples=150, deadline=None)
@given(ops)
def test_random_sequences_keep_the_heap_consistent(seq):
    lib = _lib()
    CAP = 4 << 20
    a, b = C.c_void_p(lib.bshmem_test_alloc_new(CAP)), C.c_void_p(lib.bshmem_test_alloc_new(CAP))
    backed = CAP
    live = {}  # offset -> rounded size
    try:
        for kind, x, align in seq:
            if kind == "alloc":
                off, off_b = lib.bshmem_test_alloc_malloc(a, x, align), lib.bshmem_test_alloc_malloc(b, x, align)
                assert off == off_b  # same sequence, same answer
                if off < 0:
                    continue
                assert off % max(align, 512) == 0 and off + x <= backed
                for o, sz in live.items():
                    assert off + x <= o or o + sz <= off, "ranges overlap"
                live[off] = x
            elif kind == "free" and live:
                off = sorted(live)[x % len(live)]
                assert lib.bshmem_test_alloc_free(a, off) == 0 and lib.bshmem_test_alloc_free(b, off) == 0
                del live[off]
                assert lib.bshmem_test_alloc_free(a, off) != 0  # double free is refused
            elif kind == "grow":
                lib.bshmem_test_alloc_grow(a, backed, x << 20)
                lib.bshmem_test_alloc_grow(b, backed, x << 20)
                backed += x << 20
            assert lib.bshmem_test_alloc_check(a) == 0
            assert lib.bshmem_test_alloc_digest(a) == lib.bshmem_test_alloc_digest(b)
        for off in list(live):
            assert lib.bshmem_test_alloc_free(a, off) == 0
        assert lib.bshmem_test_alloc_in_use(a) == 0
        assert lib.bshmem_test_alloc_largest_free(a) == backed  # everything coalesced back into one range
        assert lib.bshmem_test_alloc_check(a) == 0
    finally:
        lib.bshmem_test_alloc_delete(a)
        lib.bshmem_test_alloc_delete(b)
