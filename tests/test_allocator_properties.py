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


def test_sizes_whose_rounding_overflows_are_refused():
    """A size within 511 bytes of SIZE_MAX rounds up to zero: it must be refused, not recorded as a zero-length block
    that the next allocation would alias; the same for sizes beyond what the heap holds."""
    lib = _lib()
    a = C.c_void_p(lib.bshmem_test_alloc_new(1 << 20))
    try:
        for huge in ((1 << 64) - 100, (1 << 64) - 511, (1 << 64) - 512, (1 << 63), (1 << 20) + 1):
            assert lib.bshmem_test_alloc_malloc(a, huge, 0) < 0, huge
            assert lib.bshmem_test_alloc_in_use(a) == 0 and lib.bshmem_test_alloc_check(a) == 0
        first = lib.bshmem_test_alloc_malloc(a, 512, 0)
        second = lib.bshmem_test_alloc_malloc(a, 512, 0)
        assert first == 0 and second == 512
        assert lib.bshmem_test_alloc_malloc(a, 1 << 20, 0) < 0  # no longer fits
    finally:
        lib.bshmem_test_alloc_delete(a)


@settings(max_examples=300, deadline=None)
@given(st.integers(0, 1 << 40), st.sampled_from(["", "k", "K", "m", "M", "g", "G", "t", "T"]))
def test_size_parser_round_trips_every_suffix(value, suffix):
    lib = H.load()
    shift = {"": 0, "k": 10, "m": 20, "g": 30, "t": 40}[suffix.lower()]
    if value >> (63 - shift):
        return  # would overflow 64 bits
    out = C.c_ulonglong(0)
    assert lib.bshmem_test_parse_size(f"{value}{suffix}".encode(), C.byref(out)) == 0
    assert out.value == value << shift


@settings(max_examples=200, deadline=None)
@given(st.text(alphabet="0123456789kKmMgGtT.-+ xyzeinf", max_size=12))
def test_size_parser_accepts_only_a_number_with_an_optional_multiplier(text):
    """Whatever the text: accepted means it starts with a non-negative finite number, optionally followed by one of
    k/m/g/t (what follows the multiplier is ignored), and the value fits 64 bits."""
    import math
    import re
    lib = H.load()
    out = C.c_ulonglong(0)
    ok = lib.bshmem_test_parse_size(text.encode(), C.byref(out)) == 0
    m = re.match(r"\s*\+?((\d+\.?\d*|\.\d+)([eE][+-]?\d+)?)\s*([kKmMgGtT]?)", text)
    if ok:
        assert m is not None, text
        shift = {"": 0, "k": 10, "m": 20, "g": 30, "t": 40}[m.group(4).lower()]
        want = math.ceil(float(m.group(1)) * (1 << shift))
        assert want < 1 << 64 and abs(out.value - want) <= max(1, want >> 50), (text, out.value, want)
    elif m is not None and m.end() == len(text):
        # a clean number + multiplier is only refused when it does not fit
        shift = {"": 0, "k": 10, "m": 20, "g": 30, "t": 40}[m.group(4).lower()]
        assert float(m.group(1)) * (1 << shift) >= (1 << 64) * (1 - 2 ** -40), text
