"""The allocation-free MoE dispatch entry point against the ordinary one.

Some users of this library may not allocate device memory at all (a plug-in inside a serving
process with a fixed memory budget, code under a memory-accounting sandbox): they can pass their
own inputs and outputs but cannot provide the kernel's scratch block.  For them
``bshmem_moe_dispatch_local_noalloc`` keeps that block in a fixed array inside the library.  This
test calls it through its exported C symbol, twice in a row (the array keeps the previous call's
contents, so the second call proves that everything that must start at zero is cleared), and
compares with ``bshmem_moe_dispatch`` on one PE.  Row order inside an expert's segment is free in
both, so rows are compared through the slot map; everything else must be identical.

The file name sorts late on purpose: a run that stops at the first failure has then already
run the tests of everything older.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from nvshmem_b200.ops.moe import _lib, _DispatchArgs  # noqa: F401
    lib = _lib()
    lib.bshmem_moe_dispatch_local_noalloc.restype = C.c_int
    lib.bshmem_moe_dispatch_local_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.bshmem_moe_noalloc_error_bits.restype = C.c_int
    lib.bshmem_moe_noalloc_error_bits.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    return lib


def _reference(lib, x, idx, E):
    """The existing entry point with caller-allocated scratch, one PE."""
    from nvshmem_b200.ops.moe import _DispatchArgs
    T, H = x.shape
    K = idx.shape[1]
    dev = x.device
    recv = torch.zeros(T * K, H, dtype=torch.bfloat16, device=dev)
    slot = torch.full((T, K), -7, dtype=torch.int32, device=dev)
    offs = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    flags = torch.zeros(4, dtype=torch.int64, device=dev)
    scratch = torch.zeros(lib.bshmem_moe_scratch_bytes(E) // 4 + 64, dtype=torch.int32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    a = _DispatchArgs()
    a.T, a.H, a.K, a.E, a.rank, a.npes, a.payload, a.cap_rows, a.epoch = T, H, K, E, 0, 1, 0, T * K, 1
    a.error_flag, a.x, a.topk_idx = err.data_ptr(), x.data_ptr(), idx.data_ptr()
    a.recv_x[0], a.counts[0], a.flags[0] = recv.data_ptr(), counts.data_ptr(), flags.data_ptr()
    a.slot_map, a.expert_offsets, a.scratch = slot.data_ptr(), offs.data_ptr(), scratch.data_ptr()
    assert lib.bshmem_moe_dispatch(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    assert int(err) == 0
    return recv, slot, offs


def _noalloc(lib, x, idx, E, own_error_word=True):
    """`own_error_word=False` passes no error flag: the kernel's error bits then go to the word inside the built-in
    array and are read back with bshmem_moe_noalloc_error_bits."""
    T, H = x.shape
    K = idx.shape[1]
    recv = torch.zeros(T * K, H, dtype=torch.bfloat16, device=x.device)
    slot = torch.full((T, K), -7, dtype=torch.int32, device=x.device)
    offs = torch.zeros(E + 1, dtype=torch.int32, device=x.device)
    err = torch.zeros(1, dtype=torch.int32, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    st = lib.bshmem_moe_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), T, H, K, E, recv.data_ptr(), slot.data_ptr(), offs.data_ptr(),
                                               err.data_ptr() if own_error_word else None, stream)
    assert st == 0
    if own_error_word:
        torch.cuda.synchronize(x.device)
        assert int(err) == 0
    else:
        bits = C.c_int(-1)
        assert lib.bshmem_moe_noalloc_error_bits(stream, C.byref(bits)) == 0
        assert bits.value == 0
    return recv, slot, offs


def _canonical(x, idx, recv, slot, offs, E):
    """Checks one result on its own and returns, per expert, the sorted list of tokens in its segment."""
    T, K = idx.shape
    valid = idx >= 0
    tt, jj = valid.nonzero(as_tuple=True)
    rows = slot[tt, jj].long()
    assert torch.equal(slot[~valid], torch.full_like(slot[~valid], -1))
    assert int(offs[0]) == 0 and int(offs[E]) == rows.numel()
    assert rows.unique().numel() == rows.numel(), "two pairs share a row"
    assert torch.equal(recv[rows], x[tt]), "a row does not hold its token"
    e_of = idx[tt, jj].long()
    assert bool(((rows >= offs[e_of]) & (rows < offs[e_of + 1])).all()), "row outside its expert's segment"
    order = torch.argsort(e_of * T + tt)
    return e_of[order], tt[order]


def _compare_on(lib, device_index, own_error_word):
    torch.cuda.set_device(device_index)
    dev = torch.device("cuda", device_index)
    g = torch.Generator(device=dev).manual_seed(99)
    for call, (T, H, K, E) in enumerate([(300, 512, 4, 24), (257, 1024, 8, 64)]):  # two calls in a row, different sizes
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        idx = torch.rand(T, E, device=dev, generator=g).topk(K, dim=-1).indices.to(torch.int32).contiguous()
        idx[call, 0] = -1
        ref = _reference(lib, x, idx, E)
        got = _noalloc(lib, x, idx, E, own_error_word)
        assert torch.equal(got[2], ref[2]), "segment boundaries differ"
        ce_ref, ct_ref = _canonical(x, idx, *ref, E)
        ce_got, ct_got = _canonical(x, idx, *got, E)
        assert torch.equal(ce_ref, ce_got) and torch.equal(ct_ref, ct_got)


def test_noalloc_dispatch_matches_the_ordinary_entry_point_twice():
    _compare_on(_load(), 0, own_error_word=True)


def test_noalloc_dispatch_without_an_error_flag_keeps_its_error_bits_readable():
    _compare_on(_load(), 0, own_error_word=False)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_noalloc_dispatch_on_a_second_gpu_uses_that_gpus_array():
    """The array exists once per GPU and its address is looked up per GPU: the same two calls on device 1."""
    try:
        _compare_on(_load(), 1, own_error_word=True)
    finally:
        torch.cuda.set_device(0)


def test_noalloc_dispatch_refuses_sizes_beyond_its_scratch():
    lib = _load()
    torch.cuda.set_device(0)
    x = torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(8, 1, dtype=torch.int32, device="cuda")
    out = torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda")
    slot = torch.zeros(8, 1, dtype=torch.int32, device="cuda")
    offs = torch.zeros(2000, dtype=torch.int32, device="cuda")
    st = lib.bshmem_moe_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 8, 128, 1, 1025, out.data_ptr(), slot.data_ptr(), offs.data_ptr(), None,
                                               torch.cuda.current_stream().cuda_stream)
    assert st == 2  # BSHMEM_MOE_ERR_SHAPE
    # a product T * K beyond 32-bit row numbers is a shape error too, not a kernel full of overflow flags
    st = lib.bshmem_moe_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 1 << 28, 128, 16, 8, out.data_ptr(), slot.data_ptr(), offs.data_ptr(), None,
                                               torch.cuda.current_stream().cuda_stream)
    assert st == 2
