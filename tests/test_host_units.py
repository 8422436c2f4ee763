"""Unit tests of the host library's pure-CPU pieces through its C test hooks: option parsing, log and
NVTX masks, the allocator (against an interval model), and the nvshmem-info tool."""
import ctypes as C
import os
import random
import subprocess

import pytest


@pytest.fixture(scope="module")
def lib(hostlib):
    hostlib.bshmem_test_alloc_new.restype = C.c_void_p
    hostlib.bshmem_test_alloc_malloc.restype = C.c_longlong
    hostlib.bshmem_test_alloc_digest.restype = C.c_ulonglong
    hostlib.bshmem_test_alloc_in_use.restype = C.c_ulonglong
    hostlib.bshmem_test_alloc_largest_free.restype = C.c_ulonglong
    hostlib.bshmem_test_log_subsys.restype = C.c_uint
    hostlib.bshmem_test_nvtx_groups.restype = C.c_uint
    return hostlib


@pytest.mark.parametrize("text,want", [("1024", 1024), ("20m", 20 << 20), ("20M", 20 << 20), ("3.1M", 3250586), (".5m", 524288), ("0.5g", 1 << 29),
                                       ("2t", 2 << 40), ("7k", 7168), ("20kk", 20 << 10)])
def test_size_parser_accepts_suffixes(lib, text, want):
    out = C.c_ulonglong()
    assert lib.bshmem_test_parse_size(text.encode(), C.byref(out)) == 0
    assert out.value == want


@pytest.mark.parametrize("text", ["", "abc", "-5", "12q", "m"])
def test_size_parser_rejects_junk(lib, text):
    out = C.c_ulonglong()
    assert lib.bshmem_test_parse_size(text.encode(), C.byref(out)) != 0


@pytest.mark.parametrize("text,want", [("1", 1), ("true", 1), ("YES", 1), ("on", 1), ("", 1), ("0", 0), ("False", 0), ("no", 0), ("off", 0)])
def test_bool_parser(lib, text, want):
    out = C.c_int(-1)
    assert lib.bshmem_test_parse_bool(text.encode(), C.byref(out)) == 0 and out.value == want


def test_bool_parser_rejects_junk(lib):
    out = C.c_int()
    assert lib.bshmem_test_parse_bool(b"maybe", C.byref(out)) != 0


def test_log_subsystem_masks(lib):
    INIT, COLL, MEM = 1, 2, 32
    assert lib.bshmem_test_log_subsys(b"") == 0xFFFFFFFF
    assert lib.bshmem_test_log_subsys(b"INIT,COLL") == INIT | COLL
    assert lib.bshmem_test_log_subsys(b"mem") == MEM
    assert lib.bshmem_test_log_subsys(b"^MEM") == (~MEM) & 0xFFFFFFFF
    assert lib.bshmem_test_log_subsys(b"ALL") == 0xFFFFFFFF


def test_nvtx_groups(lib):
    assert lib.bshmem_test_nvtx_groups(b"off") == 0
    assert lib.bshmem_test_nvtx_groups(b"init,coll") == (1 | 8)
    assert lib.bshmem_test_nvtx_groups(b"all") == 0xFFFFFFFF
    common = lib.bshmem_test_nvtx_groups(b"common")
    assert common & 1 and common & 2 and common & 8 and not common & (1 << 11)


def test_invalid_environment_value_is_counted(lib):
    os.environ["NVSHMEM_SYMMETRIC_SIZE"] = "lots"
    try:
        assert lib.bshmem_test_options_count_bad() == 1
    finally:
        del os.environ["NVSHMEM_SYMMETRIC_SIZE"]
    assert lib.bshmem_test_options_count_bad() == 0


def test_options_dump_reflects_environment(lib):
    os.environ["NVSHMEM_MAX_TEAMS"] = "77"
    try:
        buf = C.create_string_buffer(32768)
        lib.bshmem_test_options_dump(buf, len(buf))
        text = buf.value.decode()
        assert "NVSHMEM_MAX_TEAMS=77 (set)" in text and "NVSHMEM_SYMMETRIC_SIZE=1073741824" in text
    finally:
        del os.environ["NVSHMEM_MAX_TEAMS"]


class IntervalModel:
    """Reference allocator: first fit over a sorted free list, 512-byte granule, same alignment rule."""

    def __init__(self, cap):
        self.free = [(0, cap)]
        self.used = {}

    def malloc(self, size, align):
        size = (size + 511) // 512 * 512
        align = max(align, 512)
        for i, (s, l) in enumerate(self.free):
            a = (s + align - 1) // align * align
            if a + size <= s + l:
                parts = []
                if a > s:
                    parts.append((s, a - s))
                if s + l > a + size:
                    parts.append((a + size, s + l - a - size))
                self.free[i:i + 1] = parts
                self.used[a] = size
                return a
        return -1

    def release(self, off):
        size = self.used.pop(off)
        self.free.append((off, size))
        self.free.sort()
        merged = []
        for s, l in self.free:
            if merged and merged[-1][0] + merged[-1][1] == s:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((s, l))
        self.free = merged


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_allocator_matches_interval_model(lib, seed):
    cap = 64 << 20
    h = C.c_void_p(lib.bshmem_test_alloc_new(cap))
    model = IntervalModel(cap)
    rng = random.Random(seed)
    live = []
    for step in range(600):
        if live and rng.random() < 0.45:
            off = live.pop(rng.randrange(len(live)))
            assert lib.bshmem_test_alloc_free(h, off) == 0
            model.release(off)
        else:
            size = int(2 ** rng.uniform(3, 21))
            align = rng.choice([0, 64, 256, 4096, 1 << 16])
            got = lib.bshmem_test_alloc_malloc(h, size, align)
            want = model.malloc(size, align)
            assert got == want, (step, size, align, got, want)
            if got >= 0:
                assert got % max(align, 512) == 0
                live.append(got)
        assert lib.bshmem_test_alloc_check(h) == 0
    assert lib.bshmem_test_alloc_in_use(h) == sum(model.used.values())
    assert lib.bshmem_test_alloc_free(h, 12345) != 0  # unknown offset is refused
    for off in live:
        lib.bshmem_test_alloc_free(h, off)
    assert lib.bshmem_test_alloc_largest_free(h) == cap  # everything coalesced again
    lib.bshmem_test_alloc_delete(h)


def test_allocator_history_digest_is_order_sensitive(lib):
    a, b = C.c_void_p(lib.bshmem_test_alloc_new(1 << 20)), C.c_void_p(lib.bshmem_test_alloc_new(1 << 20))
    x = lib.bshmem_test_alloc_malloc(a, 1000, 0)
    y = lib.bshmem_test_alloc_malloc(a, 2000, 0)
    y2 = lib.bshmem_test_alloc_malloc(b, 2000, 0)
    x2 = lib.bshmem_test_alloc_malloc(b, 1000, 0)
    assert (x, y) != (x2, y2)
    assert lib.bshmem_test_alloc_digest(a) != lib.bshmem_test_alloc_digest(b)
    lib.bshmem_test_alloc_delete(a)
    lib.bshmem_test_alloc_delete(b)


def test_allocator_growth_adds_adjacent_chunk(lib):
    h = C.c_void_p(lib.bshmem_test_alloc_new(1 << 20))
    assert lib.bshmem_test_alloc_malloc(h, 2 << 20, 0) == -1
    lib.bshmem_test_alloc_grow(h, 1 << 20, 3 << 20)
    assert lib.bshmem_test_alloc_malloc(h, 2 << 20, 0) == 0  # the old and the new chunk coalesced
    assert lib.bshmem_test_alloc_check(h) == 0
    lib.bshmem_test_alloc_delete(h)


def test_nvshmem_info_tool():
    from nvshmem_b200.bindings import host as H
    exe = H.lib_path("nvshmem-info")
    if not exe.exists():
        from nvshmem_b200.utils.build import build_all
        build_all(only="info")
    out = subprocess.run([str(exe), "-a"], capture_output=True, text=True, env=dict(os.environ, NVSHMEM_SYMMETRIC_SIZE="2g"))
    assert out.returncode == 0
    assert "NVSHMEM_SYMMETRIC_SIZE" in out.stdout and "2147483648" in out.stdout and "sm_100a" in out.stdout
    rst = subprocess.run([str(exe), "-e", "-r"], capture_output=True, text=True)
    assert ".. c:var:: NVSHMEM_DEBUG" in rst.stdout


def test_python_layer_imports_and_reports_version():
    import nvshmem_b200.core as nv
    v = nv.get_version()
    assert v["openshmem_spec_version"] == (1, 3) and v["libnvshmem_version"][0] == 3


def test_local_buffer_registration_table():
    """Sorted, non-overlapping table of registered local ranges (no GPU: bookkeeping only)."""
    import ctypes as C
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    lib.nvshmemx_buffer_register.argtypes = [C.c_void_p, C.c_size_t]
    lib.nvshmemx_buffer_unregister.argtypes = [C.c_void_p]
    buf = C.create_string_buffer(1 << 16)
    base = C.addressof(buf)
    assert lib.nvshmemx_buffer_register(base + 4096, 8192) == 0
    assert lib.nvshmemx_buffer_register(base + 4096, 8192) != 0          # registered twice
    assert lib.nvshmemx_buffer_register(base + 8192, 4096) != 0          # inside a registered range
    assert lib.nvshmemx_buffer_register(base, 4097) != 0                 # runs into the next range
    assert lib.nvshmemx_buffer_register(base, 4096) == 0                 # adjacent below is fine
    assert lib.nvshmemx_buffer_register(base + 12288, 4096) == 0         # adjacent above too
    assert lib.nvshmemx_buffer_register(None, 16) != 0 and lib.nvshmemx_buffer_register(base + 32768, 0) != 0
    assert lib.nvshmemx_buffer_unregister(base + 100) != 0               # not the start of a range
    assert lib.nvshmemx_buffer_unregister(base + 4096) == 0
    assert lib.nvshmemx_buffer_register(base + 6000, 100) == 0           # the hole can be used again
    lib.nvshmemx_buffer_unregister_all()
    assert lib.nvshmemx_buffer_unregister(base) != 0


def test_unique_id_with_a_foreign_version_is_refused():
    """An id made by another ABI version (or a corrupted one) is rejected before any connection is attempted."""
    import ctypes as C
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    uid = H.UniqueId()
    assert lib.nvshmemx_get_uniqueid(C.byref(uid)) == 0
    good_version = uid.version
    assert good_version == (1 << 16) + 128
    uid.version = good_version + (1 << 16)
    lib.bshmem_test_boot_init.restype = C.c_void_p
    lib.bshmem_test_boot_strerror.restype = C.c_char_p
    st = C.c_int(0)
    h = lib.bshmem_test_boot_init(C.byref(uid), 0, 1, C.byref(st))
    assert not h and st.value == 3, st.value  # BOOT_ERR_VERSION
    assert b"version" in lib.bshmem_test_boot_strerror(st.value)
    # the untouched id still works for a job of one
    uid.version = good_version
    h = lib.bshmem_test_boot_init(C.byref(uid), 0, 1, C.byref(st))
    assert h and st.value == 0
    lib.bshmem_test_boot_finalize(C.c_void_p(h))


def test_transport_seam_capabilities_and_plugin_errors(hostlib):
    """The built-in load/store transport reports no reach across hosts and full capabilities (with the same-device bit)
    for another PE on the same GPU; a transport plugin that does not exist is a clean error."""
    import ctypes as C
    caps, attr = C.c_uint(0), C.c_uint(0)
    assert hostlib.bshmem_test_transport_caps(0, 0, C.byref(caps), C.byref(attr)) == 0 and caps.value == 0
    assert attr.value == 0b111                      # no endpoints, no registration, no proxy
    assert hostlib.bshmem_test_transport_caps(1, 1, C.byref(caps), C.byref(attr)) == 0
    MAP, LD, ST, ATOM, SAME = 1, 2, 4, 8, 128
    assert caps.value & (MAP | LD | ST | ATOM | SAME) == (MAP | LD | ST | ATOM | SAME)
    assert hostlib.bshmem_test_transport_load(b"no_such_transport") != 0


def test_flat_binding_structs_are_views_of_c_memory():
    """The struct wrappers of nvshmem.bindings: defaults, field access, arrays, wrapping foreign memory."""
    import ctypes as C
    import numpy as np
    import nvshmem.bindings as b
    u = b.UniqueId(3)
    assert len(u) == 3 and list(u.version) == [(1 << 16) + 128] * 3 and u.ptr == u._data.ctypes.data
    with pytest.raises(TypeError):
        int(u)
    one = u[1]
    one.version = 7
    assert list(u.version) == [(1 << 16) + 128, 7, (1 << 16) + 128] and u[-2].version == 7  # a view, not a copy
    with pytest.raises(IndexError):
        u[3]
    raw = (C.c_char * 128)()
    w = b.UniqueId.from_ptr(C.addressof(raw))
    w.version = 0x01020304
    assert bytes(raw[:4]) == (0x01020304).to_bytes(4, "little")
    ro = b.UniqueId.from_ptr(C.addressof(raw), readonly=True)
    with pytest.raises(ValueError):
        ro.version = 1
    with pytest.raises(ValueError):
        b.UniqueId.from_ptr(0)
    cfg = b.TeamConfig()
    cfg.num_contexts, cfg.uniqueid = 2, 99
    assert (cfg.version, cfg.num_contexts, cfg.uniqueid) == ((2 << 16) + 64, 2, 99) and b.TeamConfig() != cfg and b.TeamConfig() == b.TeamConfig()
    attr = b.InitAttr()
    args = attr._data["args"][0].view(np.int32)
    assert attr.mpi_comm == 0 and args[0] == (2 << 16) + 128 and (args[6], args[7], args[8]) == (-1, -1, -1)
    assert b.Team_id.TEAM_WORLD == 0 and b.Signal_op.SIGNAL_ADD == 10 and b.Status.SUCCESS == 0
    with pytest.raises(b.NVSHMEMError):
        b.check_status(3)
    with pytest.raises(AttributeError):
        b.no_such_function
