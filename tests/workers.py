"""Worker bodies of the multi-process tests.  `python -m tests.workers <name>` runs one of them as
rank RANK of WORLD_SIZE; with BSHMEM_TEST_GPU=1 each rank uses GPU LOCAL_RANK (NCCL + VMM heap),
otherwise the gloo backend and the host-memory heap, which needs no GPU."""
from __future__ import annotations

import ctypes as C
import os
import random
import sys

import torch
import torch.distributed as dist

GPU = os.environ.get("BSHMEM_TEST_GPU") == "1"
RANK = int(os.environ.get("RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
WORKERS = {}


def worker(fn):
    WORKERS[fn.__name__] = fn
    return fn


def setup():
    import nvshmem_b200.core as nv
    if GPU:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
        nv.init(device=int(os.environ["LOCAL_RANK"]), initializer_method="torch")
    else:
        dist.init_process_group("gloo")
        nv.init(initializer_method="torch")
    return nv


def teardown(nv):
    if GPU:
        torch.cuda.synchronize()
    nv.finalize()
    dist.barrier()
    dist.destroy_process_group()


def mark(msg):
    """Progress line (the harness shows the tail of each rank's output when a worker fails)."""
    print(f"[rank {RANK}] {msg}", flush=True)


def gather_objects(obj):
    out = [None] * WORLD
    dist.all_gather_object(out, obj)
    return out


# ====================================================================== host-only (also valid on GPU)
@worker
def flat_bindings_on_host_heap():
    """The pointer-level bindings (the reference package's ``nvshmem.bindings`` names) end to end on the host-memory
    heap: unique-id initialisation through the attribute structs, allocation, peer pointers, a put with signal,
    typed collectives, a team split, finalisation.  torch only carries the unique id between the processes."""
    import ctypes as C
    import numpy as np
    import nvshmem.bindings as b
    dist.init_process_group("gloo")
    n, me = WORLD, RANK
    assert b.init_status() == b.Init_status.STATUS_NOT_INITIALIZED
    uid = b.UniqueId()
    assert len(uid) == 1 and uid.version == (1 << 16) + 128 and int(uid) == uid.ptr
    if me == 0:
        b.get_uniqueid(uid.ptr)
    raw = [bytes(uid._data.tobytes())]
    dist.broadcast_object_list(raw, src=0)
    uid = b.UniqueId.from_data(np.frombuffer(bytearray(raw[0]), dtype=b.uniqueid_dtype))
    attr = b.InitAttr()
    assert attr.version == (2 << 16) + 144
    b.set_attr_uniqueid_args(me, n, uid, attr)
    b.hostlib_init_attr(b.Flags.INIT_WITH_UNIQUEID, attr.ptr)
    assert b.init_status() >= b.Init_status.STATUS_IS_INITIALIZED
    assert (b.my_pe(), b.n_pes()) == (me, n) and b.team_n_pes(b.Team_id.TEAM_WORLD) == n
    major, minor = C.c_int(-1), C.c_int(-1)
    b.info_get_version(C.addressof(major), C.addressof(minor))
    assert major.value >= 1 and minor.value >= 0
    count = 1000
    src, dst, sig = b.malloc(4 * count), b.calloc(count * n, 4), b.calloc(1, 8)
    assert src and dst and sig and b.align(256, 1024) % 256 == 0
    mine = np.ctypeslib.as_array(C.cast(src, C.POINTER(C.c_float)), shape=(count,))
    out = np.ctypeslib.as_array(C.cast(dst, C.POINTER(C.c_float)), shape=(count * n,))
    mine[:] = np.arange(count, dtype=np.float32) + 1000 * me
    b.barrier_all()
    # typed collectives (counts in elements)
    b.float_sum_reduce_on_stream(b.Team_id.TEAM_WORLD, dst, src, count, 0)
    assert np.allclose(out[:count], n * np.arange(count) + 1000 * sum(range(n)))
    b.float_fcollect_on_stream(b.Team_id.TEAM_WORLD, dst, src, count, 0)
    assert all(np.array_equal(out[p * count:(p + 1) * count], np.arange(count, dtype=np.float32) + 1000 * p) for p in range(n))
    b.int32_broadcast_on_stream(b.Team_id.TEAM_WORLD, dst, src, count, n - 1, 0)
    assert np.array_equal(out[:count], np.arange(count, dtype=np.float32) + 1000 * (n - 1))
    try:
        b.float_sum_reduce_on_stream(12345, dst, src, count, 0)  # no such team
        raise AssertionError("a bad team handle must raise")
    except b.NVSHMEMError as e:
        assert e.status != 0
    # put with signal to the right neighbour, peer pointer of the left one
    right, left = (me + 1) % n, (me - 1) % n
    b.barrier_all()
    b.putmem_signal_on_stream(dst, src, 4 * count, sig, 7, b.Signal_op.SIGNAL_ADD, right, 0)
    b.quiet_on_stream(0)
    b.signal_wait_until_on_stream(sig, b.Cmp_type.CMP_GE, 7, 0)
    assert np.array_equal(out[:count], np.arange(count, dtype=np.float32) + 1000 * left)
    peer = b.ptr(src, left)
    assert peer and np.ctypeslib.as_array(C.cast(peer, C.POINTER(C.c_float)), shape=(count,))[5] == 5 + 1000 * left
    assert b.ptr(src, me) == src and b.mc_ptr(b.Team_id.TEAM_WORLD, src) == 0  # no multicast on host memory
    # teams: the even PEs
    cfg, new = b.TeamConfig(), C.c_int(-1)
    assert cfg.version == (2 << 16) + 64
    b.team_split_strided(b.Team_id.TEAM_WORLD, 0, 2, (n + 1) // 2, cfg.ptr, 0, C.addressof(new))
    if me % 2 == 0:
        assert new.value >= b.Team_id.TEAMS_MIN and b.team_my_pe(new.value) == me // 2
        assert b.team_translate_pe(new.value, b.team_my_pe(new.value), b.Team_id.TEAM_WORLD) == me
        b.barrier(new.value)
        b.team_destroy(new.value)
    else:
        assert new.value == b.Team_id.TEAM_INVALID
    b.barrier_all()
    for p in (src, dst, sig):
        b.free(p)
    b.hostlib_finalize()
    assert b.init_status() == b.Init_status.STATUS_NOT_INITIALIZED
    dist.barrier()
    dist.destroy_process_group()


@worker
def several_pes_per_gpu_status():
    """Host-memory heap with a pretended GPU per PE (NVSHMEM_TEST_FAKE_GPU = rank // 2, set before init): the
    same-GPU and GPU-leader teams and the LIMITED / FULL status.  MODE=none: no MPS pipe directory -> LIMITED;
    MODE=full: a directory with a control file and 50 % each -> FULL; MODE=over: 60 % each -> LIMITED."""
    import tempfile
    mode = os.environ["MPG_MODE"]
    os.environ["NVSHMEM_TEST_FAKE_GPU"] = str(RANK // 2)
    tmp = tempfile.mkdtemp()
    if mode == "none":
        os.environ["CUDA_MPS_PIPE_DIRECTORY"] = os.path.join(tmp, "absent")
    else:
        open(os.path.join(tmp, "control"), "w").close()
        os.environ["CUDA_MPS_PIPE_DIRECTORY"] = tmp
        os.environ["CUDA_MPS_ACTIVE_THREAD_PERCENTAGE"] = "50" if mode == "full" else "60"
    nv = setup()
    n, me = nv.n_pes(), nv.my_pe()
    sharers = 2 if (me // 2) * 2 + 1 < n else 1
    want = 2 if sharers == 1 else (4 if mode == "full" else 3)  # IS_INITIALIZED, FULL_MPG, LIMITED_MPG
    assert nv.init_status() == want, (me, nv.init_status(), want)
    assert nv.team_n_pes(nv.Teams.TEAM_SAME_GPU) == sharers and nv.team_my_pe(nv.Teams.TEAM_SAME_GPU) == me % 2
    leaders = (n + 1) // 2
    if me % 2 == 0:
        assert nv.team_n_pes(nv.Teams.TEAM_GPU_LEADERS) == leaders and nv.team_my_pe(nv.Teams.TEAM_GPU_LEADERS) == me // 2
    # host-initiated traffic between PEs of one GPU works in every mode
    x = nv.tensor((8,), torch.int64)
    y = nv.tensor((8,), torch.int64, zero=True)
    x.fill_(me + 1)
    nv.barrier_all()
    mate = me ^ 1 if (me ^ 1) < n else me
    nv.put(y, x, mate)
    nv.barrier_all()
    assert int(y[0]) == mate + 1
    nv.free_tensor(x)
    nv.free_tensor(y)
    teardown(nv)


@worker
def python_layer_on_host_heap():
    """The nvshmem4py-style layer end to end with no GPU: symmetric tensors over the host-memory heap, put / get /
    put-with-signal on a 'stream' (immediate on this back end), peer views, teams, tracked frees."""
    nv = setup()
    n, me = nv.n_pes(), nv.my_pe()
    assert n == WORLD and me == RANK and nv.init_status() >= 2 and nv.is_initialized()
    assert nv.team_my_pe(nv.Teams.TEAM_WORLD) == me and nv.team_n_pes(nv.Teams.TEAM_WORLD) == n
    right, left = (me + 1) % n, (me - 1) % n
    t = nv.tensor((4, 16), torch.float32, zero=True)
    assert tuple(t.shape) == (4, 16) and t.dtype == torch.float32 and float(t.abs().sum()) == 0.0
    src = torch.arange(64, dtype=torch.float32).view(4, 16) + 1000 * me
    nv.barrier_all() if GPU else H_barrier()
    nv.put(t, src, right)
    H_barrier()
    assert torch.equal(t, torch.arange(64, dtype=torch.float32).view(4, 16) + 1000 * left)
    back = torch.empty(4, 16, dtype=torch.float32)
    nv.get(back, t, right)
    assert torch.equal(back, torch.arange(64, dtype=torch.float32).view(4, 16) + 1000 * me)  # what I wrote there
    # put with signal: the signal word on the target counts arrivals
    sig = nv.tensor((1,), torch.int64, zero=True)
    H_barrier()
    nv.put_signal(t, src * 2, sig, 5, nv.SignalOp.SIGNAL_ADD, right)
    H_barrier()
    assert nv.signal_fetch(sig) == 5 and torch.equal(t, (torch.arange(64, dtype=torch.float32).view(4, 16) + 1000 * left) * 2)
    nv.signal_op(sig, 9, nv.SignalOp.SIGNAL_SET, right)
    H_barrier()
    assert nv.signal_fetch(sig) == 9
    # signal_wait really waits on this back end: the left neighbour raises my signal after a delay
    import time
    if me % 2 == 1 or n == 1:
        time.sleep(0.3)
    nv.signal_op(sig, 20, nv.SignalOp.SIGNAL_SET, right)
    nv.signal_wait(sig, 20, nv.ComparisonType.CMP_GE)
    assert nv.signal_fetch(sig) == 20 and nv.error_bits() == 0
    H_barrier()
    # a signal that nobody sends: the wait gives up after the bound and reports it
    nv.set_wait_timeout_ms(200)
    t0 = time.time()
    nv.signal_wait(sig, 1000, nv.ComparisonType.CMP_EQ)
    assert 0.15 < time.time() - t0 < 5.0 and nv.error_bits() & 1, nv.error_bits()
    nv.clear_errors()
    nv.set_wait_timeout_ms(5000)
    H_barrier()
    # typed waits on arrays: the right neighbour fills my three words one by one; negative values compare as signed
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    words = nv.tensor((3,), torch.int64, zero=True)
    H_barrier()
    for k in range(3):
        lib.nvshmem_long_p(C.c_void_p(words.data_ptr() + 8 * k), C.c_long(-5 + k), left)
    status = (C.c_int * 3)(0, 0, 0)
    lib.nvshmemx_long_wait_until_all_on_stream.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_long, C.c_void_p]
    lib.nvshmemx_long_wait_until_all_on_stream(C.c_void_p(words.data_ptr()), 3, status, int(nv.ComparisonType.CMP_LT), 0, None)
    assert words.tolist() == [-5, -4, -3] and nv.error_bits() == 0
    H_barrier()
    nv.free_tensor(words)
    # a peer view aliases the neighbour's memory (process-shared mapping on this back end)
    peer = nv.get_peer_tensor(t, right)
    assert torch.equal(peer, (torch.arange(64, dtype=torch.float32).view(4, 16) + 1000 * me) * 2)
    # A view never holds the allocation: views of every PE (the caller's own has the allocation's address) are taken
    # and dropped, and the collective free of the parent still runs on every PE.
    from nvshmem_b200.core import memory as _mem
    parent = nv.tensor((32,), torch.float32)
    views = [nv.get_peer_tensor(parent, p) for p in range(n)]
    assert views[me].data_ptr() == parent.data_ptr() and _mem._tracked[parent.data_ptr()]["ref_count"] == 1
    nv.free_tensor(views[me])
    assert parent.data_ptr() in _mem._tracked
    nv.free_tensor(parent)
    assert parent.data_ptr() not in _mem._tracked, "the parent's free was skipped because of a view"
    for p in range(n):
        if p != me:
            nv.free_tensor(views[p])
    # teams through the Python layer
    if n >= 2:
        evens = nv.team_split_strided(nv.Teams.TEAM_WORLD, 0, 2, (n + 1) // 2)
        if me % 2 == 0:
            assert nv.team_my_pe(evens) == me // 2 and nv.team_n_pes(evens) == (n + 1) // 2
            assert nv.team_translate_pe(evens, nv.team_my_pe(evens), nv.Teams.TEAM_WORLD) == me
            nv.team_destroy(evens)
        else:
            assert evens == -1 or nv.team_my_pe(evens) == -1
    # helpers of the compatibility module
    assert nv.get_size((4, 16), torch.float32) == 256 and nv.tensor_get_buffer(t).size >= 256
    assert nv.NvshmemResource().device_id == (int(os.environ["LOCAL_RANK"]) if GPU else -1)
    H_barrier()
    nv.free_tensor(sig)
    nv.free_tensor(t)
    teardown(nv)


@worker
def collectives_on_host_heap():
    """The data collectives of the Python layer with no GPU (CPU versions over the host-memory heap) against a
    local oracle: every rank can regenerate every rank's input from its seed."""
    nv = setup()
    n, me = nv.n_pes(), nv.my_pe()

    def data(rank, count, dtype):
        g = torch.Generator().manual_seed(1000 + 17 * rank + count)
        if dtype.is_floating_point:
            return (torch.rand(count, generator=g) * 2 - 0.5).to(dtype)
        return torch.randint(1, 90, (count,), generator=g).to(dtype)

    def oracle(op, stacked, dtype):
        acc = stacked.double() if dtype.is_floating_point else stacked.long()
        if op == "sum":
            out = acc.sum(0)
        elif op == "prod":
            out = acc.prod(0)
        elif op == "min":
            out = acc.min(0).values
        elif op == "max":
            out = acc.max(0).values
        else:
            out = acc[0]
            for k in range(1, acc.shape[0]):
                out = {"and": out & acc[k], "or": out | acc[k], "xor": out ^ acc[k]}[op]
        return out

    cases = [(torch.float32, "sum"), (torch.bfloat16, "sum"), (torch.float16, "max"), (torch.float64, "min"), (torch.int32, "sum"), (torch.int64, "xor"),
             (torch.uint8, "and"), (torch.int16, "or"), (torch.float32, "prod")]
    for dtype, op in cases:
        for count in (1, 7, 256, 4099):
            if op == "prod" and count > 256:
                continue
            src, dst = nv.tensor((count,), dtype), nv.tensor((count,), dtype)
            src.copy_(data(me, count, dtype))
            want = oracle(op, torch.stack([data(r, count, dtype) for r in range(n)]), dtype)
            nv.reduce(nv.Teams.TEAM_WORLD, dst, src, op)
            if dtype.is_floating_point:
                tol = {torch.bfloat16: 2 ** -6, torch.float16: 2 ** -9}.get(dtype, 1e-5) * max(1.0, float(want.abs().max()))
                assert float((dst.double() - want).abs().max()) <= tol, ("reduce", dtype, op, count)
            else:
                assert torch.equal(dst.long(), want.to(dtype).long()), ("reduce", dtype, op, count)
            work = nv.tensor((count,), dtype)
            work.copy_(data(me, count, dtype))
            nv.reduce(nv.Teams.TEAM_WORLD, work, work, op)  # in place
            assert torch.equal(work, dst), ("reduce in place", dtype, op, count)
            for t in (src, dst, work):
                nv.free_tensor(t)
    for dtype in (torch.float32, torch.int32, torch.bfloat16):
        for blk in (1, 5, 300):
            full = nv.tensor((blk * n,), dtype)
            part = nv.tensor((blk,), dtype)
            gathered = nv.tensor((blk * n,), dtype, zero=True)
            mine = data(me, blk * n, dtype)
            full.copy_(mine)
            # reducescatter: my block of the element-wise sum
            nv.reducescatter(nv.Teams.TEAM_WORLD, part, full, "sum")
            want = oracle("sum", torch.stack([data(r, blk * n, dtype) for r in range(n)]), dtype)[me * blk:(me + 1) * blk]
            tol = 2 ** -6 * max(1.0, float(want.abs().max())) if dtype == torch.bfloat16 else 1e-5 * max(1.0, float(want.abs().max()))
            assert float((part.double() - want.double()).abs().max()) <= tol, ("reducescatter", dtype, blk)
            # fcollect: everyone's first block, in rank order
            nv.fcollect(nv.Teams.TEAM_WORLD, gathered, full[:blk])
            assert torch.equal(gathered, torch.cat([data(r, blk * n, dtype)[:blk] for r in range(n)])), ("fcollect", dtype, blk)
            # alltoall: block me of every rank's buffer
            H_barrier()
            nv.alltoall(nv.Teams.TEAM_WORLD, gathered, full)
            assert torch.equal(gathered, torch.cat([data(r, blk * n, dtype)[me * blk:(me + 1) * blk] for r in range(n)])), ("alltoall", dtype, blk)
            # broadcast from the last rank
            H_barrier()
            nv.broadcast(nv.Teams.TEAM_WORLD, gathered, full, root=n - 1)
            assert torch.equal(gathered, data(n - 1, blk * n, dtype)), ("broadcast", dtype, blk)
            H_barrier()
            for t in (full, part, gathered):
                nv.free_tensor(t)
    # a sub-team: the even ranks reduce among themselves
    if n >= 3:
        evens = nv.team_split_strided(nv.Teams.TEAM_WORLD, 0, 2, (n + 1) // 2)
        v = nv.tensor((8,), torch.float32)
        out = nv.tensor((8,), torch.float32)
        v.fill_(float(me + 1))
        H_barrier()
        if me % 2 == 0:
            nv.reduce(evens, out, v, "sum")
            assert float(out[0]) == float(sum(r + 1 for r in range(0, n, 2)))
            nv.team_destroy(evens)
        H_barrier()
        nv.free_tensor(v)
        nv.free_tensor(out)
    # the typed C entry points (blocking and "on stream") reach the same CPU code
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    a32, b32 = nv.tensor((5,), torch.int32), nv.tensor((5,), torch.int32)
    a32.copy_(torch.arange(5, dtype=torch.int32) + me)
    H_barrier()
    assert lib.nvshmem_int_sum_reduce(0, C.c_void_p(b32.data_ptr()), C.c_void_p(a32.data_ptr()), C.c_size_t(5)) == 0
    assert b32.tolist() == [n * k + n * (n - 1) // 2 for k in range(5)]
    assert lib.nvshmemx_int_max_reduce_on_stream(0, C.c_void_p(b32.data_ptr()), C.c_void_p(a32.data_ptr()), C.c_size_t(5), None) == 0
    assert b32.tolist() == [k + n - 1 for k in range(5)]
    H_barrier()
    nv.free_tensor(a32)
    nv.free_tensor(b32)
    assert nv.error_bits() == 0
    teardown(nv)


@worker
def typed_host_api_all_types():
    """Every RMA type name of the API through its host entry points (p, g, put, get, iput, iget, put_nbi + quiet) on the
    host-memory heap: checks the generated type tables (names, element sizes, strides), not the transport."""
    nv = setup()
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    n, me = nv.n_pes(), nv.my_pe()
    right, left = (me + 1) % n, (me - 1) % n
    types = {"char": C.c_char, "schar": C.c_byte, "short": C.c_short, "int": C.c_int, "long": C.c_long, "longlong": C.c_longlong, "uchar": C.c_ubyte,
             "ushort": C.c_ushort, "uint": C.c_uint, "ulong": C.c_ulong, "ulonglong": C.c_ulonglong, "int8": C.c_int8, "int16": C.c_int16, "int32": C.c_int32,
             "int64": C.c_int64, "uint8": C.c_uint8, "uint16": C.c_uint16, "uint32": C.c_uint32, "uint64": C.c_uint64, "size": C.c_size_t, "ptrdiff": C.c_ssize_t,
             "float": C.c_float, "double": C.c_double, "half": C.c_uint16, "bfloat16": C.c_uint16}
    lib.nvshmem_malloc.restype = C.c_void_p
    for name, ct in types.items():
        es = C.sizeof(ct)
        count = 12
        sym = lib.nvshmem_calloc(2 * count, es)
        assert sym
        Arr = ct * count
        raw16 = name in ("half", "bfloat16")  # passed through as bit patterns
        def val(rank, k):
            v = (rank * 13 + k * 3 + 1) % 100
            return bytes([v]) if name == "char" else (float(v) if name in ("float", "double") else v)
        mine = Arr(*[val(me, k) for k in range(count)])
        # put to the right neighbour's first half; get it back
        getattr(lib, f"nvshmem_{name}_put")(C.c_void_p(sym), mine, C.c_size_t(count), right)
        lib.nvshmem_barrier_all()
        local = (ct * (2 * count)).from_address(sym)
        assert [local[k] for k in range(count)] == [val(left, k) for k in range(count)], (name, "put")
        back = Arr()
        getattr(lib, f"nvshmem_{name}_get")(back, C.c_void_p(sym), C.c_size_t(count), right)
        assert list(back) == [val(me, k) for k in range(count)], (name, "get")
        # strided: every second element of mine into every third slot of the right neighbour's second half
        lib.nvshmem_barrier_all()
        fn = getattr(lib, f"nvshmem_{name}_iput")
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_ssize_t, C.c_ssize_t, C.c_size_t, C.c_int]
        fn(C.c_void_p(sym + count * es), mine, 3, 2, 4, right)
        lib.nvshmem_barrier_all()
        assert [local[count + 3 * k] for k in range(4)] == [val(left, 2 * k) for k in range(4)], (name, "iput")
        got = (ct * 4)()
        fn = getattr(lib, f"nvshmem_{name}_iget")
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_ssize_t, C.c_ssize_t, C.c_size_t, C.c_int]
        fn(got, C.c_void_p(sym + count * es), 1, 3, 4, right)
        assert list(got) == [val(me, 2 * k) for k in range(4)], (name, "iget")
        # non-blocking put + quiet, and the scalar forms (not for the 16-bit floating types, whose scalars are structs)
        lib.nvshmem_barrier_all()
        getattr(lib, f"nvshmem_{name}_put_nbi")(C.c_void_p(sym), mine, C.c_size_t(count), left)
        lib.nvshmem_quiet()
        lib.nvshmem_barrier_all()
        assert [local[k] for k in range(count)] == [val(right, k) for k in range(count)], (name, "put_nbi")
        if not raw16:
            p, g = getattr(lib, f"nvshmem_{name}_p"), getattr(lib, f"nvshmem_{name}_g")
            p.argtypes, g.argtypes, g.restype = [C.c_void_p, ct, C.c_int], [C.c_void_p, C.c_int], ct
            lib.nvshmem_barrier_all()
            p(C.c_void_p(sym), val(me, 5), right)
            lib.nvshmem_barrier_all()
            assert local[0] == val(left, 5), (name, "p")
            assert g(C.c_void_p(sym), right) == val(me, 5), (name, "g")
        lib.nvshmem_barrier_all()
        lib.nvshmem_free(C.c_void_p(sym))
    # sized forms: 8 .. 128 bits
    for bits in (8, 16, 32, 64, 128):
        es, count = bits // 8, 6
        sym = lib.nvshmem_calloc(count, es)
        src = bytes([(me * 31 + k) % 251 for k in range(count * es)])
        getattr(lib, f"nvshmem_put{bits}")(C.c_void_p(sym), src, C.c_size_t(count), right)
        lib.nvshmem_barrier_all()
        assert C.string_at(sym, count * es) == bytes([(left * 31 + k) % 251 for k in range(count * es)]), bits
        back = C.create_string_buffer(count * es)
        getattr(lib, f"nvshmem_get{bits}")(back, C.c_void_p(sym), C.c_size_t(count), right)
        assert back.raw == src, bits
        lib.nvshmem_barrier_all()
        lib.nvshmem_free(C.c_void_p(sym))
    teardown(nv)


@worker
def host_atomics_all_types():
    """Every atomic of the API for every type class through the host entry points: all PEs hammer one word on PE 0
    (add / inc / fetch forms must not lose updates), then bitwise and exchange forms with known outcomes."""
    nv = setup()
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    n, me = nv.n_pes(), nv.my_pe()
    bitwise = {"uint": C.c_uint, "ulong": C.c_ulong, "ulonglong": C.c_ulonglong, "int32": C.c_int32, "uint32": C.c_uint32, "int64": C.c_int64, "uint64": C.c_uint64}
    standard = dict(bitwise, int=C.c_int, long=C.c_long, longlong=C.c_longlong, size=C.c_size_t, ptrdiff=C.c_ssize_t)
    extended = dict(standard, float=C.c_float, double=C.c_double)
    lib.nvshmem_calloc.restype = C.c_void_p

    def fn(name, res, *args):
        f = getattr(lib, name)
        f.restype, f.argtypes = res, list(args)
        return f

    for tname, ct in standard.items():
        word = lib.nvshmem_calloc(2, 8)
        tgt = C.c_void_p(word)
        iters = 25
        lib.nvshmem_barrier_all()
        seen = set()
        for _ in range(iters):
            fn(f"nvshmem_{tname}_atomic_inc", None, C.c_void_p, C.c_int)(tgt, 0)
            fn(f"nvshmem_{tname}_atomic_add", None, C.c_void_p, ct, C.c_int)(tgt, 2, 0)
            seen.add(fn(f"nvshmem_{tname}_atomic_fetch_inc", ct, C.c_void_p, C.c_int)(tgt, 0))
            seen.add(fn(f"nvshmem_{tname}_atomic_fetch_add", ct, C.c_void_p, ct, C.c_int)(tgt, 3, 0))
        lib.nvshmem_barrier_all()
        total = fn(f"nvshmem_{tname}_atomic_fetch", ct, C.c_void_p, C.c_int)(tgt, 0)
        assert total == n * iters * 7, (tname, total)
        assert len(seen) == 2 * iters, (tname, "fetch forms returned a value twice")  # every fetched value is a distinct moment
        # compare-and-swap: exactly one PE wins the race from the known value
        lib.nvshmem_barrier_all()
        old = fn(f"nvshmem_{tname}_atomic_compare_swap", ct, C.c_void_p, ct, ct, C.c_int)(tgt, n * iters * 7, 1000 + me, 0)
        winners = gather_objects(old == n * iters * 7)
        assert sum(winners) == 1, (tname, winners)
        lib.nvshmem_barrier_all()
        lib.nvshmem_free(tgt)
    for tname, ct in extended.items():
        word = lib.nvshmem_calloc(2, 8)
        tgt = C.c_void_p(word)
        lib.nvshmem_barrier_all()
        fn(f"nvshmem_{tname}_atomic_set", None, C.c_void_p, ct, C.c_int)(tgt, 40 + me, (me + 1) % n)
        lib.nvshmem_barrier_all()
        left = (me - 1) % n
        assert fn(f"nvshmem_{tname}_atomic_fetch", ct, C.c_void_p, C.c_int)(tgt, me) == 40 + left, tname
        prev = fn(f"nvshmem_{tname}_atomic_swap", ct, C.c_void_p, ct, C.c_int)(tgt, 90 + me, me)
        assert prev == 40 + left, tname
        lib.nvshmem_barrier_all()
        lib.nvshmem_free(tgt)
    for tname, ct in bitwise.items():
        word = lib.nvshmem_calloc(2, 8)
        tgt = C.c_void_p(word)
        lib.nvshmem_barrier_all()
        fn(f"nvshmem_{tname}_atomic_or", None, C.c_void_p, ct, C.c_int)(tgt, 1 << me, 0)       # every PE sets its bit on PE 0
        lib.nvshmem_barrier_all()
        allbits = (1 << n) - 1
        assert fn(f"nvshmem_{tname}_atomic_fetch", ct, C.c_void_p, C.c_int)(tgt, 0) == allbits, tname
        lib.nvshmem_barrier_all()
        before = fn(f"nvshmem_{tname}_atomic_fetch_xor", ct, C.c_void_p, ct, C.c_int)(tgt, 1 << me, 0)  # and clears it again
        assert before & (1 << me), tname
        lib.nvshmem_barrier_all()
        assert fn(f"nvshmem_{tname}_atomic_fetch", ct, C.c_void_p, C.c_int)(tgt, 0) == 0, tname
        lib.nvshmem_barrier_all()
        if me == 0:
            fn(f"nvshmem_{tname}_atomic_set", None, C.c_void_p, ct, C.c_int)(tgt, 0xFF, 0)
        lib.nvshmem_barrier_all()
        fn(f"nvshmem_{tname}_atomic_and", None, C.c_void_p, ct, C.c_int)(tgt, 0xFF ^ (1 << me), 0)
        lib.nvshmem_barrier_all()
        assert fn(f"nvshmem_{tname}_atomic_fetch_and", ct, C.c_void_p, ct, C.c_int)(tgt, 0xFF, 0) == 0xFF ^ allbits, tname
        got = fn(f"nvshmem_{tname}_atomic_fetch_or", ct, C.c_void_p, ct, C.c_int)(tgt, 0, 0)
        assert got == 0xFF ^ allbits, tname
        lib.nvshmem_barrier_all()
        lib.nvshmem_free(tgt)
    teardown(nv)


def H_barrier():
    from nvshmem_b200.bindings import host as H
    if GPU:
        torch.cuda.synchronize()
    H.load().nvshmem_barrier_all()


@worker
def alloc_symmetry():
    """Seeded 64-call malloc/align/free sequence: every PE must see identical offsets."""
    nv = setup()
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    rng = random.Random(20240611)
    base = lib.nvshmemx_b200_heap_info(0)
    live, trace = [], []
    for i in range(64):
        if live and rng.random() < 0.4:
            p = live.pop(rng.randrange(len(live)))
            lib.nvshmem_free(p)
            trace.append(("free", p - base))
        else:
            size = int(2 ** rng.uniform(3, 24))
            align = rng.choice([64, 256, 4096])
            p = lib.nvshmem_align(align, size)
            assert p and (p - base) % max(align, 512) == 0, (i, size, align, p)
            live.append(p)
            trace.append(("alloc", p - base, size, align))
    traces = gather_objects(trace)
    assert all(t == traces[0] for t in traces), "offsets differ between PEs"
    digests = gather_objects(lib.nvshmemx_b200_heap_info(6))
    assert len(set(digests)) == 1
    for p in live:
        lib.nvshmem_free(p)
    lib.nvshmem_barrier_all()
    teardown(nv)


@worker
def host_rma_and_atomics():
    nv = setup()
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    n = WORLD
    buf = lib.nvshmem_calloc(4096, 8)
    right, left = (RANK + 1) % n, (RANK - 1) % n
    src = (C.c_long * 8)(*[RANK * 100 + k for k in range(8)])
    lib.nvshmem_putmem(buf, src, 64, right)
    lib.nvshmem_barrier_all()
    got = (C.c_long * 8)()
    lib.nvshmem_getmem(got, buf, 64, RANK)
    assert list(got) == [left * 100 + k for k in range(8)], list(got)
    # get from the right neighbour: it holds what I wrote
    lib.nvshmem_getmem(got, buf, 64, right)
    assert list(got) == [RANK * 100 + k for k in range(8)]
    # p / g
    lib.nvshmem_long_p(buf + 1024, 7000 + RANK, right)
    lib.nvshmem_barrier_all()
    assert lib.nvshmem_long_g(buf + 1024, RANK) == 7000 + left
    # strided: every 2nd source element into every 3rd slot on the left neighbour
    strided = (C.c_long * 8)(*range(10, 18))
    lib.nvshmem_long_iput(buf + 2048, strided, 3, 2, 4, left)
    lib.nvshmem_barrier_all()
    lib.nvshmem_getmem(got, buf + 2048, 64, RANK)
    assert [got[0], got[3], got[6]] == [10, 12, 14]
    # atomics on PE 0
    lib.nvshmem_barrier_all()
    old = lib.nvshmem_long_atomic_fetch_add(buf + 3072, RANK + 1, 0)
    olds = gather_objects(old)
    lib.nvshmem_barrier_all()
    total = lib.nvshmem_long_atomic_fetch(buf + 3072, 0)
    assert total == n * (n + 1) // 2, total
    assert sorted(olds)[0] == 0 and len(set(olds)) == n
    winner = lib.nvshmem_long_atomic_compare_swap(buf + 3080, 0, RANK + 1, 0)
    winners = gather_objects(winner)
    assert winners.count(0) == 1
    mask = lib.nvshmem_uint64_atomic_fetch_or(buf + 3088, 1 << RANK, 0)
    lib.nvshmem_barrier_all()
    assert lib.nvshmem_uint64_atomic_fetch_or(buf + 3088, 0, 0) == (1 << n) - 1
    # signals from the host
    sig = lib.nvshmem_calloc(1, 8)
    stream = torch.cuda.current_stream().cuda_stream if GPU else 0
    lib.nvshmemx_signal_op_on_stream(sig, 5, H.SIGNAL_SET, right, stream)
    lib.nvshmemx_signal_op_on_stream(sig, 2, H.SIGNAL_ADD, right, stream)
    if GPU:
        torch.cuda.synchronize()
    lib.nvshmem_barrier_all()
    assert lib.nvshmem_signal_fetch(sig) == 7
    lib.nvshmem_free(sig)
    lib.nvshmem_free(buf)
    teardown(nv)


@worker
def teams():
    nv = setup()
    n = WORLD
    T = nv.Teams
    assert nv.team_my_pe(T.TEAM_WORLD) == RANK and nv.team_n_pes(T.TEAM_WORLD) == n
    assert nv.team_n_pes(T.TEAM_NODE) == n and nv.team_n_pes(T.TEAM_SHARED) == n
    assert nv.team_n_pes(T.TEAM_SAME_MYPE_NODE) == 1
    # even PEs
    even = nv.team_split_strided(T.TEAM_WORLD, 0, 2, (n + 1) // 2)
    if RANK % 2 == 0:
        assert even >= 6 and nv.team_my_pe(even) == RANK // 2 and nv.team_n_pes(even) == (n + 1) // 2
        assert nv.team_translate_pe(even, nv.team_my_pe(even), T.TEAM_WORLD) == RANK
        assert nv.team_translate_pe(T.TEAM_WORLD, RANK, even) == RANK // 2
        if n > 1:
            assert nv.team_translate_pe(T.TEAM_WORLD, 1, even) == -1
        from nvshmem_b200.bindings import host as H
        assert H.load().nvshmem_team_sync(even) == 0
    else:
        assert even == T.TEAM_INVALID
    # create/destroy loop: slots are recycled
    seen = set()
    for _ in range(6):
        t = nv.team_split_strided(T.TEAM_WORLD, 0, 1, n)
        seen.add(t)
        nv.team_destroy(t)
    assert len(seen) <= 2
    if RANK % 2 == 0:
        nv.team_destroy(even)
    # 2-D split
    if n >= 4:
        xt, yt = nv.team_split_2d(T.TEAM_WORLD, 2)
        assert nv.team_n_pes(xt) == min(2, n - (RANK // 2) * 2) and nv.team_my_pe(xt) == RANK % 2
        assert nv.team_my_pe(yt) == RANK // 2
        nv.team_destroy(xt)
        nv.team_destroy(yt)
    # unique-id team of the odd PEs (arbitrary membership)
    if n >= 3:
        from nvshmem_b200.bindings import host as H
        uid = gather_objects(nv.get_team_unique_id())[0]
        members = [p for p in range(n) if p % 2 == 1]
        cfg = H.TeamConfig(uniqueid=uid)
        if RANK in members:
            t = nv.team_init(cfg, 0, len(members), members.index(RANK))
            assert nv.team_n_pes(t) == len(members) and nv.team_translate_pe(t, members.index(RANK), T.TEAM_WORLD) == RANK
            nv.team_destroy(t)
        else:
            assert nv.team_init(cfg, 0, 0, -1) == T.TEAM_INVALID
    nv.barrier_all() if GPU else None
    teardown(nv)


@worker
def bootstrap_raw():
    """The UID bootstrap alone (no heap): allgather / alltoall / barrier with odd sizes."""
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    dist.init_process_group("gloo")
    payload = [None]
    if RANK == 0:
        uid = H.UniqueId()
        assert lib.nvshmemx_get_uniqueid(C.byref(uid)) == 0
        payload = [uid.to_bytes()]
    dist.broadcast_object_list(payload, src=0)
    uid = H.UniqueId.from_bytes(payload[0])
    lib.bshmem_test_boot_init.restype = C.c_void_p
    st = C.c_int(-1)
    h = lib.bshmem_test_boot_init(C.byref(uid), RANK, WORLD, C.byref(st))
    assert h and st.value == 0, st.value
    h = C.c_void_p(h)
    for nbytes in (1, 8, 33, 4096, 300000):
        send = bytes([(RANK * 7 + i) % 251 for i in range(nbytes)])
        recv = C.create_string_buffer(nbytes * WORLD)
        assert lib.bshmem_test_boot_allgather(h, send, recv, nbytes) == 0
        for r in range(WORLD):
            assert recv.raw[r * nbytes:(r + 1) * nbytes] == bytes([(r * 7 + i) % 251 for i in range(nbytes)]), (nbytes, r)
        a2a_send = b"".join(bytes([(RANK * 16 + p + i) % 256 for i in range(nbytes)]) for p in range(WORLD))
        a2a_recv = C.create_string_buffer(nbytes * WORLD)
        assert lib.bshmem_test_boot_alltoall(h, a2a_send, a2a_recv, nbytes) == 0
        for p in range(WORLD):
            assert a2a_recv.raw[p * nbytes:(p + 1) * nbytes] == bytes([(p * 16 + RANK + i) % 256 for i in range(nbytes)]), (nbytes, p)
        assert lib.bshmem_test_boot_barrier(h) == 0
    mn, nn = C.c_int(), C.c_int()
    lib.bshmem_test_boot_node_info(h, C.byref(mn), C.byref(nn))
    assert nn.value == WORLD and mn.value == RANK
    lib.bshmem_test_boot_finalize(h)
    dist.barrier()
    dist.destroy_process_group()


@worker
def bootstrap_missing_rank():
    """Host-side fault injection: the root drops the last rank's registration, so nobody gets an
    address table; every rank's init returns a time-out status within the bound, none exits or hangs."""
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    dist.init_process_group("gloo")
    payload = [None]
    if RANK == 0:
        lib.bshmem_test_boot_drop_rank(WORLD - 1)
        uid = H.UniqueId()
        assert lib.nvshmemx_get_uniqueid(C.byref(uid)) == 0
        payload = [uid.to_bytes()]
    dist.broadcast_object_list(payload, src=0)
    uid = H.UniqueId.from_bytes(payload[0])
    lib.bshmem_test_boot_init.restype = C.c_void_p
    lib.bshmem_test_boot_strerror.restype = C.c_char_p
    st = C.c_int(-1)
    h = lib.bshmem_test_boot_init(C.byref(uid), RANK, WORLD, C.byref(st))
    assert not h and st.value in (2, 5), (st.value, lib.bshmem_test_boot_strerror(st.value))
    dist.barrier()
    dist.destroy_process_group()


@worker
def rank_never_joins():
    """One rank never calls init: the others get a time-out status from init (short bound) and carry on."""
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    dist.init_process_group("gloo")
    payload = [None]
    if RANK == 0:
        uid = H.UniqueId()
        assert lib.nvshmemx_get_uniqueid(C.byref(uid)) == 0
        payload = [uid.to_bytes()]
    dist.broadcast_object_list(payload, src=0)
    if RANK != WORLD - 1:
        uid = H.UniqueId.from_bytes(payload[0])
        st = lib.nvshmemx_b200_init_uid(C.byref(uid), RANK, WORLD, -1)
        assert st != 0
        assert lib.nvshmemx_init_status() != 2
    dist.barrier()
    dist.destroy_process_group()


# ====================================================================== GPU: device API
def _devtest():
    from nvshmem_b200.bindings import host as H
    H.load()
    lib = C.CDLL(str(H.lib_path("libbshmem_devtest.so")))
    H.load().nvshmemx_b200_module_sync()  # the library was loaded after init: hand it the device state
    assert lib.devtest_preload() == 0
    return lib


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@worker
def device_rma():
    nv = setup()
    dt = _devtest()
    n = WORLD
    right = (RANK + 1) % n
    cap = 1 << 16
    dst = nv.tensor((cap,), torch.uint8)
    srcsym = nv.tensor((cap,), torch.uint8)
    local = torch.empty(cap, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(77 + RANK)
    sizes = list(range(1, 40)) + [63, 64, 65, 127, 128, 129, 255, 256, 257, 1000, 4096, 4097, 30001]
    for scope in (0, 1, 2):
        for nbi in (0, 1):
            for size in (sizes if scope == 2 else sizes[::3]):
                for off_d, off_s in ((0, 0), (1, 1), (3, 5), (16, 8), (8, 16)):
                    if size + max(off_d, off_s) > cap:
                        continue
                    local.random_(0, 256, generator=g)
                    dst.zero_()
                    nv.barrier_all()
                    assert dt.devtest_put(C.c_void_p(dst.data_ptr() + off_d), C.c_void_p(local.data_ptr() + off_s), C.c_size_t(size), right, scope, nbi, _stream()) == 0
                    nv.barrier_all()
                    torch.cuda.synchronize()
                    # what landed here came from the left neighbour: compare through a gather of sources
                    want = [torch.empty_like(local) for _ in range(n)]
                    dist.all_gather(want, local)
                    left = (RANK - 1) % n
                    assert torch.equal(dst[off_d:off_d + size], want[left][off_s:off_s + size]), (scope, nbi, size, off_d, off_s)
                    assert int(dst[off_d + size:off_d + size + 8].sum()) == 0 and (off_d == 0 or int(dst[:off_d].sum()) == 0), "wrote outside the target range"
    # get: pull from the right neighbour's symmetric buffer
    for scope in (0, 1, 2):
        for size in (1, 7, 64, 257, 4097, 30001):
            srcsym.random_(0, 256, generator=g)
            local.zero_()
            nv.barrier_all()
            assert dt.devtest_get(C.c_void_p(local.data_ptr()), C.c_void_p(srcsym.data_ptr()), C.c_size_t(size), right, scope, 0, _stream()) == 0
            torch.cuda.synchronize()
            want = [torch.empty_like(srcsym) for _ in range(n)]
            dist.all_gather(want, srcsym)
            assert torch.equal(local[:size], want[right][:size]), (scope, size)
            nv.barrier_all()
    # typed calls
    nelem = 1024
    fdst, idst, ddst, hdst = nv.tensor((nelem,), torch.float32), nv.tensor((4,), torch.int32), nv.tensor((nelem,), torch.float64, zero=True), nv.tensor((nelem,), torch.bfloat16)
    fsrc = torch.rand(nelem, device="cuda") + RANK
    dsrc = torch.arange(nelem, device="cuda", dtype=torch.float64) + 1000 * RANK
    hsrc = (torch.rand(nelem, device="cuda") + RANK).to(torch.bfloat16)
    gout = torch.zeros(4, dtype=torch.int32, device="cuda")
    nv.barrier_all()
    assert dt.devtest_typed(C.c_void_p(fdst.data_ptr()), C.c_void_p(fsrc.data_ptr()), C.c_void_p(idst.data_ptr()), C.c_void_p(ddst.data_ptr()), C.c_void_p(dsrc.data_ptr()),
                            C.c_void_p(hdst.data_ptr()), C.c_void_p(hsrc.data_ptr()), C.c_size_t(nelem), right, C.c_void_p(gout.data_ptr()), _stream()) == 0
    nv.barrier_all()
    torch.cuda.synchronize()
    left = (RANK - 1) % n
    fs = [torch.empty_like(fsrc) for _ in range(n)]
    dist.all_gather(fs, fsrc)
    hs = [torch.empty_like(hsrc) for _ in range(n)]
    dist.all_gather(hs, hsrc)
    assert torch.equal(fdst, fs[left]) and torch.equal(hdst, hs[left])
    assert int(idst[0]) == 1000 + left
    want_d = torch.zeros(nelem, dtype=torch.float64)
    want_d[0:2 * (nelem // 4):2] = (torch.arange(nelem, dtype=torch.float64) + 1000 * left)[0:3 * (nelem // 4):3]
    assert torch.equal(ddst.cpu(), want_d)
    assert gout.tolist() == [1000 + RANK, n, 1, 1], gout.tolist()
    assert nv.error_bits() == 0
    for t in (dst, srcsym, fdst, idst, ddst, hdst):
        nv.free_tensor(t)
    teardown(nv)


@worker
def device_signals_amo_barrier():
    nv = setup()
    dt = _devtest()
    n = WORLD
    right, left = (RANK + 1) % n, (RANK - 1) % n
    words = 1 << 16
    data = nv.tensor((words,), torch.int32, zero=True)
    sig = nv.tensor((2,), torch.int64, zero=True)
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    side = torch.cuda.Stream()
    for it, (scope, op) in enumerate([(0, 9), (1, 9), (2, 9), (2, 10)]):
        payload = torch.randint(0, 1 << 20, (words,), dtype=torch.int32, device="cuda")
        want_val = it + 1 if op == 9 else 3 + 3
        # consumer first, on a side stream: it spins (bounded) until the producer's signal lands
        with torch.cuda.stream(side):
            assert dt.devtest_signal_wait_sum(C.c_void_p(data.data_ptr()), C.c_size_t(words), C.c_void_p(sig.data_ptr()), 5, C.c_uint64(want_val), C.c_void_p(out.data_ptr()),
                                              C.c_void_p(side.cuda_stream)) == 0
        assert dt.devtest_put_signal(C.c_void_p(data.data_ptr()), C.c_void_p(payload.data_ptr()), C.c_size_t(words * 4), C.c_void_p(sig.data_ptr()),
                                     C.c_uint64(it + 1 if op == 9 else 3), op, right, scope, _stream()) == 0
        torch.cuda.synchronize()
        sums = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(n)]
        dist.all_gather(sums, payload.to(torch.int64).sum().reshape(1))
        assert int(out[0]) == int(sums[left]), (scope, op)
        nv.barrier_all()
    mark('signals ok')
    # ring of put_signal
    token = nv.tensor((1,), torch.int64, zero=True)
    rsig = nv.tensor((1,), torch.int64, zero=True)
    nv.barrier_all()
    rounds = 5
    assert dt.devtest_ring(C.c_void_p(token.data_ptr()), C.c_void_p(rsig.data_ptr()), rounds, C.c_uint64(0), _stream()) == 0
    torch.cuda.synchronize()
    nv.barrier_all()
    torch.cuda.synchronize()
    if RANK == 0:
        assert int(token[0]) == rounds * n * (n + 1) // 2, int(token[0])
    mark('ring ok')
    # atomics: fetch_add from every thread of every PE onto PE 0
    target = nv.tensor((4,), torch.int64, zero=True)
    ctas, threads = 4, 128
    olds = torch.zeros(ctas * threads, dtype=torch.int64, device="cuda")
    nv.barrier_all()
    assert dt.devtest_amo_fetch_add(C.c_void_p(target.data_ptr()), 0, C.c_void_p(olds.data_ptr()), ctas, threads, _stream()) == 0
    torch.cuda.synchronize()
    nv.barrier_all()
    allolds = [torch.zeros_like(olds) for _ in range(n)]
    dist.all_gather(allolds, olds)
    if RANK == 0:
        assert int(target[0]) == n * ctas * threads
        assert torch.equal(torch.cat(allolds).sort().values.cpu(), torch.arange(n * ctas * threads))
    mark('fetch_add ok')
    # mixed atomics
    t64 = nv.tensor((4,), torch.int64, zero=True)
    t32 = nv.tensor((4,), torch.int32, zero=True)
    tf = nv.tensor((2,), torch.float32, zero=True)
    t64[1] = 0x0f
    t64[2] = -1
    mixout = torch.zeros(4, dtype=torch.int64, device="cuda")
    nv.barrier_all()
    assert dt.devtest_amo_mix(C.c_void_p(t64.data_ptr()), C.c_void_p(t32.data_ptr()), C.c_void_p(tf.data_ptr()), 0, C.c_void_p(mixout.data_ptr()), _stream()) == 0
    torch.cuda.synchronize()
    nv.barrier_all()
    cas = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(n)]
    dist.all_gather(cas, mixout[1:2].clone())
    if RANK == 0:
        assert int(t64[0]) == (1 << n) - 1
        assert int(t32[0]) == 4 * n
        assert [int(c) for c in cas].count(0) == 1 and 77 <= int(t32[1]) < 77 + n
        assert int(t64[1]) == (0x0f ^ 0xff if n % 2 else 0x0f)
        assert int(t64[2]) & ((1 << n) - 1) == 0
        assert 1.5 <= float(tf[0]) < 1.5 + n
    mark('mixed atomics ok')
    # barriers in every scope with data hand-off
    slots = nv.tensor((max(n, 2),), torch.int64, zero=True)
    errs = torch.zeros(1, dtype=torch.int32, device="cuda")
    for scope in (0, 1, 2, 3):
        nv.barrier_all()
        assert dt.devtest_barrier_rounds(C.c_void_p(slots.data_ptr()), 20, scope, C.c_void_p(errs.data_ptr()), _stream()) == 0
        torch.cuda.synchronize()
        assert int(errs[0]) == 0, (scope, int(errs[0]))
        mark(f'barrier scope {scope} ok')
    assert nv.error_bits() == 0
    # bounded wait: nobody sets this flag; the kernel must return and report
    nv.set_wait_timeout_ms(300)
    nv.clear_errors()
    never = nv.tensor((1,), torch.int64, zero=True)
    res = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert dt.devtest_wait_never(C.c_void_p(never.data_ptr()), C.c_uint64(42), C.c_void_p(res.data_ptr()), _stream()) == 0
    torch.cuda.synchronize()
    assert int(res[0]) != 0 and nv.error_bits() & 1
    info = nv.direct.timeout_info()
    assert info["count"] >= 1 and info["expected"] == 42
    nv.clear_errors()
    nv.set_wait_timeout_ms(30000)
    nv.barrier_all()
    teardown(nv)


def _oracle(op, tensors):
    st = torch.stack([t.double() if t.is_floating_point() else t.long() for t in tensors])
    if op == "sum":
        return st.sum(0)
    if op == "prod":
        return st.prod(0)
    if op == "min":
        return st.min(0).values
    if op == "max":
        return st.max(0).values
    out = st[0].clone()
    for t in st[1:]:
        out = out & t if op == "and" else out | t if op == "or" else out ^ t
    return out


def _gather(t):
    """all_gather through a byte view: NCCL has no 16-bit integer type."""
    if not dist.is_initialized():
        return [t.clone()]
    raw = t.clone().contiguous().view(torch.uint8)
    outs = [torch.empty_like(raw) for _ in range(WORLD)]
    dist.all_gather(outs, raw)
    return [o.view(t.dtype).view(t.shape) for o in outs]


def _close(got, want, dtype):
    if dtype in (torch.float32, torch.float64):
        return torch.allclose(got.double(), want, rtol=1e-5, atol=1e-5)
    if dtype in (torch.float16, torch.bfloat16):
        return torch.allclose(got.double(), want, rtol=2e-2, atol=2e-2)
    return torch.equal(got.long(), want.long())


@worker
def allreduce_recursive_exchange():
    """Every member exchanges with log2(n) partners; teams of 3, 5, 6 or 7 members fold the members beyond the largest
    power of two in first.  World team and, with four or more PEs, a three-member sub-team; called several times in a
    row (the two scratch halves alternate).  Allocation and the oracle's gather involve every PE, the reduction only
    the team's members."""
    nv = setup()
    n = WORLD
    g = torch.Generator(device="cuda").manual_seed(17 + RANK)
    teams = [(0, list(range(n)))]
    sub = None
    if n >= 4:
        sub = nv.team_split_strided(0, 0, 1, 3)
        teams.append((sub, [0, 1, 2]))
    for team, members in teams:
        member = RANK in members
        for dtype, op in ((torch.float32, "sum"), (torch.int32, "max"), (torch.bfloat16, "sum"), (torch.float64, "prod"), (torch.int64, "xor")):
            for count in (1, 7, 256, 1000, 4096):
                src, dst, work = nv.tensor((count,), dtype), nv.tensor((count,), dtype), nv.tensor((count,), dtype)
                for it in range(4):  # the last pass is in place
                    if dtype.is_floating_point:
                        scale = 1.0 if op != "prod" else 0.2
                        src.copy_(((torch.rand(count, device="cuda", generator=g) * 2 - 1) * scale + (1.0 if op == "prod" else 0.0)).to(dtype))
                    else:
                        src.copy_(torch.randint(0, 1 << 12, (count,), device="cuda", generator=g).to(dtype))
                    allsrc = _gather(src)
                    want = _oracle(op, [allsrc[m] for m in members])
                    dst.zero_()
                    work.copy_(src)
                    nv.barrier_all()
                    if member:
                        if it < 3:
                            nv.reduce(team, dst, src, op, algo="recexch")
                        else:
                            nv.reduce(team, work, work, op, algo="recexch")
                        torch.cuda.synchronize()
                        got = dst if it < 3 else work
                        assert _close(got, want, dtype), ("recexch", team != 0, dtype, op, count, it, (got.double() - want.double()).abs().max().item())
                for t in (src, dst, work):
                    nv.free_tensor(t)
    if sub is not None and RANK in (0, 1, 2):
        nv.team_destroy(sub)
    assert nv.error_bits() == 0
    teardown(nv)


@worker
def collectives_on_stream():
    nv = setup()
    n = WORLD
    nvls = nv.heap_info()["mc_base"] != 0
    g = torch.Generator(device="cuda").manual_seed(5 + RANK)
    sizes = [1, 3, 8, 30, 255, 1022, 1024, 4097, 8190, 65536, 1 << 20]  # 30 floats: one 120-byte packet; 1022, 8190: a partly filled last packet
    cases = [(torch.float32, "sum"), (torch.bfloat16, "sum"), (torch.float16, "max"), (torch.int32, "min"), (torch.int64, "xor"), (torch.float64, "prod"), (torch.uint8, "and"),
             (torch.int16, "or")]
    red_algos = ["auto", "oneshot", "twoshot", "ll", "ll128"] + (["nvls_oneshot", "nvls_twoshot"] if nvls else [])
    for dtype, op in cases:
        for count in sizes:
            if dtype.is_floating_point:
                scale = 1.0 if op != "prod" else 0.2
                make = lambda m: ((torch.rand(m, device="cuda", generator=g) * 2 - 1) * scale + (1.0 if op == "prod" else 0.0)).to(dtype)
            else:
                hi = 100 if dtype in (torch.uint8,) else 1 << 12
                make = lambda m: torch.randint(0, hi, (m,), device="cuda", generator=g).to(dtype)
            src = nv.tensor((count,), dtype)
            dst = nv.tensor((count,), dtype)
            src.copy_(make(count))
            allsrc = _gather(src)
            want = _oracle(op, allsrc)
            for algo in red_algos:  # the NVLS algorithms cover float sums and 4- / 8-byte integer operators; other cases fall back
                dst.zero_()
                nv.barrier_all()
                nv.reduce(0, dst, src, op, algo=algo)
                torch.cuda.synchronize()
                assert _close(dst, want, dtype), ("reduce", dtype, op, count, algo, (dst.double() - want.double()).abs().max().item())
            # in place
            work = nv.tensor((count,), dtype)
            work.copy_(src)
            nv.barrier_all()
            nv.reduce(0, work, work, op)
            torch.cuda.synchronize()
            assert _close(work, want, dtype), ("reduce in place", dtype, op, count)
            for t in (src, dst, work):
                nv.free_tensor(t)
    # reducescatter / fcollect / alltoall / broadcast
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        for count in (1, 5, 30, 256, 2046, 4099, 1 << 18):
            make = (lambda m: (torch.rand(m, device="cuda", generator=g) * 2 - 1).to(dtype)) if dtype.is_floating_point else (lambda m: torch.randint(0, 1000, (m,), device="cuda", generator=g).to(dtype))
            big = nv.tensor((count * n,), dtype)
            small = nv.tensor((count,), dtype)
            out_big = nv.tensor((count * n,), dtype)
            big.copy_(make(count * n))
            small.copy_(make(count))
            allbig = _gather(big)
            allsmall = _gather(small)
            for algo in ["auto", "pull"] + (["nvls"] if nvls else []):
                res = nv.tensor((count,), dtype)
                nv.barrier_all()
                nv.reducescatter(0, res, big, "sum", algo=algo)
                torch.cuda.synchronize()
                want = _oracle("sum", [b[RANK * count:(RANK + 1) * count] for b in allbig])
                assert _close(res, want, dtype), ("reducescatter", dtype, count, algo)
                nv.free_tensor(res)
            for algo in ["auto", "push", "ll", "ll128"] + (["nvls"] if nvls else []):
                out_big.zero_()
                nv.barrier_all()
                nv.fcollect(0, out_big, small, algo=algo)
                torch.cuda.synchronize()
                assert torch.equal(out_big, torch.cat(allsmall)), ("fcollect", dtype, count, algo)
            out_big.zero_()
            nv.barrier_all()
            nv.alltoall(0, out_big, big)
            torch.cuda.synchronize()
            want = torch.cat([b[RANK * count:(RANK + 1) * count] for b in allbig])
            assert torch.equal(out_big, want), ("alltoall", dtype, count)
            for root in {0, n - 1}:
                for algo in ["auto", "push", "pull", "ll", "ll"] + (["nvls"] if nvls else []):  # "ll" twice: generations alternate halves
                    res = nv.tensor((count,), dtype, zero=True)
                    nv.barrier_all()
                    nv.broadcast(0, res, small, root=root, algo=algo)
                    torch.cuda.synchronize()
                    assert torch.equal(res, allsmall[root]), ("broadcast", dtype, count, root, algo)
                    nv.free_tensor(res)
            for t in (big, small, out_big):
                nv.free_tensor(t)
    # sub-team collective
    if n >= 4:
        even = nv.team_split_strided(0, 0, 2, n // 2)
        x = nv.tensor((1000,), torch.float32)
        y = nv.tensor((1000,), torch.float32)
        x.fill_(float(RANK + 1))
        nv.barrier_all()
        if RANK % 2 == 0 and RANK // 2 < n // 2:
            nv.reduce(even, y, x, "sum")
            torch.cuda.synchronize()
            assert float(y[0]) == sum(r + 1 for r in range(0, n, 2))
            nv.team_destroy(even)
        nv.barrier_all()
        nv.free_tensor(x)
        nv.free_tensor(y)
    # maxloc
    pair = nv.tensor((2,), torch.float64)
    res = nv.tensor((2,), torch.float64)
    pair[0] = float((RANK * 7) % n)
    pair[1] = float(RANK)
    nv.barrier_all()
    nv.maxloc(0, res, pair)
    torch.cuda.synchronize()
    vals = [(r * 7) % n for r in range(n)]
    assert res[0].item() == max(vals) and int(res[1].item()) == vals.index(max(vals))
    assert nv.error_bits() == 0
    teardown(nv)


@worker
def collectives_in_graph():
    """On-stream collectives captured into a CUDA graph and replayed."""
    nv = setup()
    n = WORLD
    src = nv.tensor((1 << 16,), torch.float32)
    dst = nv.tensor((1 << 16,), torch.float32)
    src.fill_(1.0 + RANK)
    nv.barrier_all()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        nv.reduce(0, dst, src, "sum", stream=s)  # warm-up outside capture
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            nv.reduce(0, dst, src, "sum", stream=s)
            nv.barrier_all(stream=s)
    for it in range(3):
        src.fill_(1.0 + RANK + it)
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        assert float(dst[123]) == sum(1.0 + r + it for r in range(n)), (it, float(dst[123]))
    teardown(nv)


@worker
def device_collectives_and_tiles():
    nv = setup()
    dt = _devtest()
    n = WORLD
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    count = 3000
    def run(kind, dst, src, cnt, root=0, threads=256):
        nv.barrier_all()
        assert dt.devtest_device_coll(kind, 0, C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), C.c_size_t(cnt), root, C.c_void_p(status.data_ptr()), threads, _stream()) == 0
        torch.cuda.synchronize()
        assert int(status[0]) == 0
    f_src, f_dst = nv.tensor((count * n,), torch.float32), nv.tensor((count * n,), torch.float32)
    f_src.copy_(torch.arange(count * n, device="cuda", dtype=torch.float32) % 13 + RANK)
    run(0, f_dst, f_src, count)
    base = torch.arange(count * n, dtype=torch.float32) % 13
    assert torch.equal(f_dst[:count].cpu(), base[:count] * n + sum(range(n)))
    run(2, f_dst, f_src, count)
    assert torch.equal(f_dst[:count].cpu(), base[RANK * count:(RANK + 1) * count] * n + sum(range(n)))
    i_src, i_dst = nv.tensor((count * n,), torch.int32), nv.tensor((count * n,), torch.int32)
    i_src.copy_((torch.arange(count * n, device="cuda") * (RANK + 3)) % 1009)
    run(1, i_dst, i_src, count)
    want = torch.stack([(torch.arange(count) * (r + 3)) % 1009 for r in range(n)]).max(0).values
    assert torch.equal(i_dst[:count].cpu().long(), want)
    for kind in (3, 8):
        i_dst.zero_()
        run(kind, i_dst, i_src, 100 if kind == 8 else count)
        m = 100 if kind == 8 else count
        want = torch.cat([((torch.arange(count * n) * (r + 3)) % 1009)[:m] for r in range(n)])
        assert torch.equal(i_dst[:m * n].cpu().long(), want), kind
    run(4, i_dst, i_src, count)
    want = torch.cat([((torch.arange(count * n) * (r + 3)) % 1009)[RANK * count:(RANK + 1) * count] for r in range(n)])
    assert torch.equal(i_dst.cpu().long(), want)
    run(5, i_dst, i_src, count, root=n - 1)
    assert torch.equal(i_dst[:count].cpu().long(), ((torch.arange(count * n) * (n - 1 + 3)) % 1009)[:count])
    h_src, h_dst = nv.tensor((4096,), torch.bfloat16), nv.tensor((4096,), torch.bfloat16)
    h_src.fill_(0.5 + RANK)
    run(6, h_dst, h_src, 4096)
    assert float(h_dst[17]) == sum(0.5 + r for r in range(n))
    u_src, u_dst = nv.tensor((512,), torch.int64), nv.tensor((512,), torch.int64)
    u_src.fill_(1 << RANK)
    run(7, u_dst, u_src, 512)
    assert int(u_dst[5]) == (1 << n) - 1
    # tiles
    R, Cc = 100, 96
    t_src, t_dst = nv.tensor((R, Cc), torch.float32), nv.tensor((R, Cc), torch.float32, zero=True)
    t_src.copy_(torch.arange(R * Cc, device="cuda", dtype=torch.float32).reshape(R, Cc) * (RANK + 1))
    for algo, (r0, c0, rows, cols) in ((1, (8, 16, 32, 64)), (2, (64, 32, 64, 64)), (1, (3, 5, 7, 9))):
        t_dst.zero_()
        nv.barrier_all()
        assert dt.devtest_tile_allreduce(0, C.c_void_p(t_dst.data_ptr()), C.c_void_p(t_src.data_ptr()), R, Cc, r0, c0, rows, cols, algo, n - 1, _stream()) == 0
        torch.cuda.synchronize()
        want = torch.zeros(R, Cc)
        r1, c1 = min(r0 + rows, R), min(c0 + cols, Cc)
        want[r0:r1, c0:c1] = (torch.arange(R * Cc, dtype=torch.float32).reshape(R, Cc) * (n * (n + 1) // 2))[r0:r1, c0:c1]
        assert torch.equal(t_dst.cpu(), want), (algo, r0, c0)
    # several CTAs at once, each with its own tile and its own row of sync flags
    for algo in (1, 2):
        t_dst.zero_()
        nv.barrier_all()
        assert dt.devtest_tile_allreduce_multi(0, C.c_void_p(t_dst.data_ptr()), C.c_void_p(t_src.data_ptr()), R, Cc, 4, 16, 24, 64, algo, 0, 4, _stream()) == 0
        torch.cuda.synchronize()
        want = torch.zeros(R, Cc)
        want[4:100, 16:80] = (torch.arange(R * Cc, dtype=torch.float32).reshape(R, Cc) * (n * (n + 1) // 2))[4:100, 16:80]
        assert torch.equal(t_dst.cpu(), want), ("multi-CTA tile reduce", algo)
    right = (RANK + 1) % n
    t_dst.zero_()
    nv.barrier_all()
    assert dt.devtest_tile_put_get(C.c_void_p(t_dst.data_ptr()), C.c_void_p(t_src.data_ptr()), R, Cc, 10, 8, 16, 32, right, 0, _stream()) == 0
    nv.barrier_all()
    torch.cuda.synchronize()
    left = (RANK - 1) % n
    want = torch.zeros(R, Cc)
    want[10:26, 8:40] = (torch.arange(R * Cc, dtype=torch.float32).reshape(R, Cc) * (left + 1))[10:26, 8:40]
    assert torch.equal(t_dst.cpu(), want)
    assert nv.error_bits() == 0
    teardown(nv)


def _moe_check(nv, payload, T, H, K, E, seed, dedup=False):
    """Dispatch + combine against a gather-based oracle; returns nothing, asserts."""
    from nvshmem_b200.ops.moe import MoeDispatchCombine
    from nvshmem_b200.ops import fused_gemm as fg
    n = WORLD
    EL = E // n
    g = torch.Generator(device="cuda").manual_seed(seed + RANK)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    probs = logits.softmax(-1)
    w, idx = probs.topk(K, dim=-1)
    idx = idx.to(torch.int32).contiguous()
    idx[0, 0] = -1  # a dropped slot must be skipped everywhere
    w = w.float().contiguous()
    moe = MoeDispatchCombine(T, H, K, E, payload=payload, wait_limit_ms=5000, dedup=dedup)
    assert moe.dedup == (dedup and n > 1)
    for it in range(2):
        recv, offs = moe.dispatch(x, idx)
        torch.cuda.synchronize()
        fg.check_errors()
        allx, allidx, allmap = _gather(x), _gather(idx), _gather(moe.slot_map)
        offs_h = offs.cpu().tolist()
        # segment sizes: expert_offsets must equal the number of pairs routed to each local expert
        for le in range(EL):
            want = sum(int((ai == RANK * EL + le).sum()) for ai in allidx)
            assert offs_h[le + 1] - offs_h[le] == want, (le, offs_h[le + 1] - offs_h[le], want)
        rows = offs_h[EL]
        got = moe.dequantized(rows) if payload == "fp8" else recv[:rows].float()
        seen = torch.zeros(rows, dtype=torch.int32, device="cuda")
        for s in range(n):
            mine = (allidx[s] >= RANK * EL) & (allidx[s] < (RANK + 1) * EL)
            tt, jj = mine.nonzero(as_tuple=True)
            r = allmap[s][tt, jj].long()
            assert int(r.min()) >= 0 and int(r.max()) < rows
            e_of_row = allidx[s][tt, jj].long() - RANK * EL
            lo = torch.tensor(offs_h, device="cuda")[e_of_row]
            hi = torch.tensor(offs_h, device="cuda")[e_of_row + 1]
            assert bool(((r >= lo) & (r < hi)).all()), "row outside its expert's segment"
            seen.index_add_(0, r, torch.ones_like(r, dtype=torch.int32))
            src_rows = allx[s][tt].float()
            if payload == "fp8":
                amax = src_rows.view(-1, H // 128, 128).abs().amax(-1, keepdim=True).expand(-1, -1, 128).reshape(-1, H)
                assert bool(((got[r] - src_rows).abs() <= 0.0625 * src_rows.abs() + amax / 448 + 1e-6).all()), "fp8 payload outside quantisation error"
            else:
                assert torch.equal(got[r], src_rows), ("payload mismatch", s)
        assert bool((seen == 1).all()), "a receive row was written twice or never"
        assert int(moe.slot_map[0, 0]) == -1
        # expert "MLP": scale by (local expert + 1)
        le_of_row = torch.bucketize(torch.arange(rows, device="cuda"), torch.tensor(offs_h[1:], device="cuda"), right=True)
        src_for_y = got if payload == "fp8" else recv[:rows].float()
        moe.expert_out[:rows] = (src_for_y * (le_of_row + 1).unsqueeze(1)).to(torch.bfloat16)
        out = moe.combine(idx, w)
        torch.cuda.synchronize()
        fg.check_errors()
        valid = (idx >= 0).float()
        factor = ((idx % EL + 1).float() * w * valid).sum(1, keepdim=True)
        want = x.float() * factor
        tol = 0.09 if payload == "fp8" else 0.02
        assert bool(((out.float() - want).abs() <= tol * want.abs() + tol * want.abs().max()).all()), (payload, (out.float() - want).abs().max().item())
        x = (x.float() * 0.5 + 0.25).to(torch.bfloat16)  # next iteration: other data, same object (epochs)
    moe.close()


@worker
def moe_dispatch_combine():
    nv = setup()
    n = WORLD
    _moe_check(nv, "bf16", T=64, H=256, K=2, E=4 * n, seed=1)
    _moe_check(nv, "bf16", T=512, H=1024, K=8, E=32 * n if n <= 4 else 256, seed=2)
    _moe_check(nv, "fp8", T=256, H=512, K=4, E=8 * n, seed=3)
    _moe_check(nv, "fp8", T=384, H=7168, K=8, E=16 * n, seed=4)
    teardown(nv)


@worker
def moe_dispatch_once_per_pe():
    """A token crosses NVLink once per destination PE and is replicated by the receiver; same oracle as above."""
    nv = setup()
    n = WORLD
    _moe_check(nv, "bf16", T=64, H=256, K=4, E=2 * n, seed=11, dedup=True)   # two experts per PE, top-4: many repeats per PE
    _moe_check(nv, "bf16", T=512, H=1024, K=8, E=32 * n if n <= 4 else 256, seed=12, dedup=True)
    _moe_check(nv, "fp8", T=256, H=512, K=4, E=8 * n, seed=13, dedup=True)
    _moe_check(nv, "fp8", T=384, H=7168, K=8, E=16 * n, seed=14, dedup=True)
    teardown(nv)


# ====================================================================== GPU: fused kernels
@worker
def fused_gemm_collectives():
    nv = setup()
    from nvshmem_b200.ops import fused_gemm as fg
    n = WORLD
    torch.manual_seed(100)
    paths_seen = []
    for (M, N, Kl) in ((128 * n, 256, 64), (256 * n, 512, 192), (1024 * n, 768, 256), (384 * n, 2048, 128)):
        xs = [(torch.randn(M, Kl, device="cuda")).to(torch.bfloat16) for _ in range(n)]   # same seed on all ranks: everyone knows all inputs
        ws = [(torch.randn(N, Kl, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(n)]
        full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
        tol = full.abs().max().item() * 2 ** -6 + 1e-2
        rows = M // n
        # With a multicast window both paths are checked: partials reduced inside the switch, and pushed partials.
        for use_mc in (True, False):
            rs = fg.GemmReduceScatter(M, N, mode="rs", wait_limit_ms=5000, use_multicast=use_mc)
            if not use_mc and paths_seen and not paths_seen[-1]:
                rs.close()
                break  # no multicast window: the first pass already was the push path
            paths_seen.append(rs.switch_path)
            for it in range(4):  # several calls: epochs and the two generations of partial-tile storage
                scale = 1.0 + it
                out = rs((xs[RANK].float() * scale).to(torch.bfloat16), ws[RANK])
                torch.cuda.synchronize()
                fg.check_errors()
                err = (out.float() - scale * full[RANK * rows:(RANK + 1) * rows]).abs().max().item()
                assert err <= tol * scale, ("rs", use_mc, M, N, Kl, it, err, tol)
            rs.close()
            ar = fg.GemmReduceScatter(M, N, mode="ar", wait_limit_ms=5000, use_multicast=use_mc)
            assert ar.switch_path == paths_seen[-1]
            for it in range(3):
                scale = 1.0 + it
                out = ar((xs[RANK].float() * scale).to(torch.bfloat16), ws[RANK])
                nv.barrier_all()
                torch.cuda.synchronize()
                fg.check_errors()
                err = (out.float() - scale * full).abs().max().item()
                assert err <= tol * scale, ("ar", use_mc, M, N, Kl, it, err, tol)
            ar.close()
    if os.environ.get("BSHMEM_EXPECT_SWITCH_PATH") == "1":
        assert any(paths_seen), "the heap has no multicast window: the switch path did not run"
    for (M, K, Nl) in ((128 * n, 64, 256), (256 * n, 512, 512), (1024 * n, 1024, 256), (384 * n, 8192, 256)):
        x_full = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(Nl, K, device="cuda") * 0.05).to(torch.bfloat16)
        rows = M // n
        for ce in (True, False):  # shard pushed by copy engines on a side stream, and by two warps of every CTA
            ag = fg.AllGatherGemm(M, K, wait_limit_ms=5000, copy_engine=ce)
            for it in range(3):
                xi = (x_full.float() * (it + 1)).to(torch.bfloat16)
                ag.shard.copy_(xi[RANK * rows:(RANK + 1) * rows])
                out = ag(w)
                torch.cuda.synchronize()
                fg.check_errors()
                ref = xi.float() @ w.float().t()
                err = (out.float() - ref).abs().max().item()
                assert err <= ref.abs().max().item() * 2 ** -7 + 1e-3, ("ag", ce, M, K, Nl, it, err)
                assert torch.equal(ag.gathered, xi), "gathered activations differ"
            ag.close()
    teardown(nv)


@worker
def tp_mlp_matches_single_device():
    nv = setup()
    from nvshmem_b200.models.tp_mlp import TensorParallelMLP
    from nvshmem_b200.ops import fused_gemm as fg
    n = WORLD
    hidden, ffn, tokens = 512, 1024 * n if n > 1 else 1024, 256 * n
    torch.manual_seed(7)  # identical full weights on every rank
    w_up = (torch.randn(ffn, hidden, device="cuda") * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(hidden, ffn, device="cuda") * 0.02).to(torch.bfloat16)
    x_full = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    mlp = TensorParallelMLP(hidden, ffn, tokens)
    fl, rows = ffn // n, tokens // n
    with torch.no_grad():
        mlp.up.weight.copy_(w_up[RANK * fl:(RANK + 1) * fl])
        mlp.down.weight.copy_(w_down[:, RANK * fl:(RANK + 1) * fl])
    x = x_full[RANK * rows:(RANK + 1) * rows].clone().requires_grad_(True)
    y = mlp(x)
    y.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    fg.check_errors()
    ref = mlp.reference(x_full, w_up, w_down)
    err = (y.float() - ref[RANK * rows:(RANK + 1) * rows]).abs().max().item()
    assert err <= 0.03 * ref.abs().max().item() + 1e-2, err
    # gradients against fp32 autograd on the full problem
    x32 = x_full.float().requires_grad_(True)
    w1, w2 = w_up.float().requires_grad_(True), w_down.float().requires_grad_(True)
    yr = torch.nn.functional.gelu(x32 @ w1.t(), approximate="tanh") @ w2.t()
    # each rank's loss is the mean over ITS rows; the sum of the ranks' losses is n * global mean
    (yr.pow(2).mean() * n).backward()
    for got, want in ((x.grad, x32.grad[RANK * rows:(RANK + 1) * rows]), (mlp.up.weight.grad, w1.grad[RANK * fl:(RANK + 1) * fl]), (mlp.down.weight.grad, w2.grad[:, RANK * fl:(RANK + 1) * fl])):
        denom = want.abs().max().item() + 1e-12
        assert (got.float() - want).abs().max().item() / denom < 0.08, (got.float() - want).abs().max().item() / denom
    mlp.close()
    teardown(nv)


@worker
def tp_mlp_stack_matches_fp32_reference():
    """The forward-only stack (fused GELU, reduce-scatter written into the next block's all-gather shard) against plain
    fp32 torch on the full problem, twice in a row on new inputs (buffers are reused between calls)."""
    nv = setup()
    from nvshmem_b200.models.tp_mlp import TensorParallelMLPStack
    from nvshmem_b200.ops import fused_gemm as fg
    n = WORLD
    hidden, ffn, tokens, layers = 512, 256 * n, 256 * n, 3
    stack = TensorParallelMLPStack(hidden, ffn, tokens, layers, init_std=0.05, seed=11 + RANK)
    assert stack.kernels_per_forward == layers * (3 if n > 1 else 2)
    fl, rows = ffn // n, tokens // n
    w_up = [torch.cat(_gather(w), 0) for w in stack.w_up]           # [ffn, hidden]: rank r holds rows r*fl..
    w_down = [torch.cat(_gather(w), 1) for w in stack.w_down]       # [hidden, ffn]: rank r holds columns r*fl..
    for it in range(2):
        torch.manual_seed(31 + it)
        x_full = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
        stack.input_shard.copy_(x_full[RANK * rows:(RANK + 1) * rows])
        y = stack()
        torch.cuda.synchronize()
        fg.check_errors()
        ref = stack.reference(x_full, w_up, w_down)[RANK * rows:(RANK + 1) * rows]
        err = (y.float() - ref).abs().max().item()
        assert err <= 0.04 * ref.abs().max().item() + 1e-2, (it, err, ref.abs().max().item())
    stack.close()
    teardown(nv)


@worker
def team_multicast_windows():
    """Teams that do not span the world get an NVLink multicast window of their own: the NVLS algorithms run on a
    strided split and on both teams of a 2-D split, and nvshmemx_mc_ptr gives a team-specific address."""
    nv = setup()
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    n, me = WORLD, RANK
    assert nv.heap_info()["mc_base"] != 0, "this test needs NVLS"
    probe = nv.tensor((4096,), torch.float32)
    world_mc = lib.nvshmemx_mc_ptr(0, C.c_void_p(probe.data_ptr()))
    assert world_mc
    teams = []
    evens = nv.team_split_strided(nv.Teams.TEAM_WORLD, 0, 2, n // 2)
    if me % 2 == 0:
        teams.append(("evens", evens, list(range(0, n, 2))))
    xt, yt = nv.team_split_2d(nv.Teams.TEAM_WORLD, 2)
    teams.append(("x", xt, [me - me % 2, me - me % 2 + 1]))
    teams.append(("y", yt, list(range(me % 2, n, 2))))
    g = torch.Generator(device="cuda").manual_seed(77 + me)
    count = 8192
    src = nv.tensor((count,), torch.float32)
    dst = nv.tensor((count,), torch.float32)
    big = nv.tensor((count * n,), torch.float32)
    src.copy_(torch.rand(count, device="cuda", generator=g) * 2 - 1)
    big.copy_(torch.rand(count * n, device="cuda", generator=g) * 2 - 1)
    allsrc, allbig = _gather(src), _gather(big)
    nv.barrier_all()
    for name, team, members in teams:
        size = len(members)
        if size < 2:
            continue
        tme = members.index(me)
        mc = lib.nvshmemx_mc_ptr(int(team), C.c_void_p(probe.data_ptr()))
        assert mc and mc != world_mc, (name, mc, world_mc)
        for algo in ("nvls_oneshot", "nvls_twoshot", "auto"):
            dst.zero_()
            nv.barrier(team)
            nv.reduce(team, dst, src, "sum", algo=algo)
            torch.cuda.synchronize()
            want = _oracle("sum", [allsrc[m] for m in members])
            assert _close(dst, want, torch.float32), ("reduce", name, algo, (dst - want).abs().max().item())
        res = nv.tensor((count,), torch.float32) if False else dst  # reuse: allocation is a world collective
        res.zero_()
        nv.barrier(team)
        nv.reducescatter(team, res, big, "sum", algo="nvls")
        torch.cuda.synchronize()
        want = _oracle("sum", [allbig[m][tme * count:(tme + 1) * count] for m in members])
        assert _close(res, want, torch.float32), ("reducescatter", name)
        out = big  # gather target: size * count elements fit
        keep = big.clone()
        nv.barrier(team)
        nv.fcollect(team, out, src, algo="nvls")
        torch.cuda.synchronize()
        assert torch.equal(out[:size * count], torch.cat([allsrc[m] for m in members])), ("fcollect", name)
        nv.barrier(team)
        nv.broadcast(team, dst, src, root=size - 1, algo="nvls")
        torch.cuda.synchronize()
        assert torch.equal(dst, allsrc[members[-1]]), ("broadcast", name)
        big.copy_(keep)
        torch.cuda.synchronize()
        nv.barrier(team)
    assert nv.error_bits() == 0
    nv.barrier_all()
    for name, team, members in teams:
        pass
    # destruction is collective over the team's members: everyone destroys its own teams in the same order
    if me % 2 == 0:
        nv.team_destroy(evens)
    nv.team_destroy(xt)
    nv.team_destroy(yt)
    # the slots (and the multicast windows) can be made again
    again = nv.team_split_strided(nv.Teams.TEAM_WORLD, 1, 2, n // 2)
    if me % 2 == 1:
        assert lib.nvshmemx_mc_ptr(int(again), C.c_void_p(probe.data_ptr()))
        nv.team_destroy(again)
    for t in (src, dst, big, probe):
        nv.free_tensor(t)
    teardown(nv)


@worker
def device_api_wrappers_and_copy_engine_collectives():
    """(1) One kernel that calls each family of thin device wrappers once: the queue-pair forms, sized puts, byte
    collectives at thread / warp / block scope.  (2) The copy-engine variants of fcollect / alltoall / broadcast on
    several PEs (one memcpy per member into the member's window, then a barrier)."""
    nv = setup()
    dt = _devtest()
    n, me = WORLD, RANK
    right, left = (me + 1) % n, (me - 1) % n
    words = 64 + 2 * n + 8
    buf = nv.tensor((words,), torch.int64, zero=True)
    sig = nv.tensor((1,), torch.int64, zero=True)
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    buf[40:48] = torch.arange(8, device="cuda", dtype=torch.int64) + 1000 * (me + 1)   # source of the block / warp puts
    buf[48] = 7000 + me                                                                # contribution to the byte collectives
    nv.barrier_all()
    torch.cuda.synchronize()
    assert dt.devtest_api_wrappers(C.c_void_p(buf.data_ptr()), C.c_void_p(sig.data_ptr()), right, C.c_void_p(status.data_ptr()), _stream()) == 0
    nv.barrier_all()
    torch.cuda.synchronize()
    got = buf.cpu().tolist()
    assert status.tolist()[0] == 0 and nv.error_bits() == 0
    assert got[0] == 101 and got[1:3] == [202, 203] and got[3:5] == [202, 203] and got[5:7] == [202, 203]      # written by my left neighbour
    assert got[7] == 202 and got[8] == 202
    src_left = [1000 * (left + 1) + i for i in range(8)]
    assert got[16:24] == src_left and got[24:32] == src_left
    assert int(sig[0]) == 7                                                             # put_signal added 5, signal_op added 2
    assert got[64:64 + n] == [7000 + p for p in range(n)]                               # fcollectmem
    assert got[49] == 7000                                                              # broadcastmem from PE 0
    assert got[64 + n:64 + 2 * n] == [7000 + me] * n                                    # alltoallmem: word `me` of every PE's gathered row
    assert status.tolist()[1] == 7000 + right                                           # qp g
    # ---- copy-engine collectives
    cnt = 1 << 16
    src, dst = nv.tensor((cnt * n,), torch.float32), nv.tensor((cnt * n,), torch.float32)
    src.copy_(torch.arange(cnt * n, device="cuda", dtype=torch.float32) + 1e6 * me)
    allsrc = _gather(src)
    nv.set_ce_collectives(1)
    try:
        dst.zero_()
        nv.barrier_all()
        nv.fcollect(0, dst, src[:cnt])
        nv.barrier_all()
        torch.cuda.synchronize()
        assert torch.equal(dst, torch.cat([a[:cnt] for a in allsrc])), "copy-engine fcollect"
        dst.zero_()
        nv.barrier_all()
        nv.alltoall(0, dst, src)
        nv.barrier_all()
        torch.cuda.synchronize()
        assert torch.equal(dst, torch.cat([a[me * cnt:(me + 1) * cnt] for a in allsrc])), "copy-engine alltoall"
        dst.zero_()
        nv.barrier_all()
        nv.broadcast(0, dst, src, root=n - 1)
        nv.barrier_all()
        torch.cuda.synchronize()
        assert torch.equal(dst, allsrc[n - 1]), "copy-engine broadcast"
    finally:
        nv.set_ce_collectives(0)
    assert nv.error_bits() == 0
    for t in (buf, sig, src, dst):
        nv.free_tensor(t)
    teardown(nv)


@worker
def device_module_via_driver_api():
    """Device code in a separately loaded module: a kernel is compiled to a cubin with nvcc, loaded with cuModuleLoadData,
    handed the library state with nvshmemx_cumodule_init, and puts to the next PE."""
    import subprocess
    import tempfile
    nv = setup()
    from nvshmem_b200.bindings import host as H
    from nvshmem_b200.utils.build import CSRC, nvcc
    lib = H.load()
    n, me = WORLD, RANK
    src_file = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "device_module_kernel.cu")
    with tempfile.TemporaryDirectory() as tmp:
        cubin = os.path.join(tmp, f"module_{me}.cubin")
        subprocess.run([nvcc(), "-cubin", "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(CSRC / "include"), "-o", cubin, src_file], check=True)
        image = open(cubin, "rb").read()
    cu = C.CDLL("libcuda.so.1")
    mod, fn = C.c_void_p(), C.c_void_p()
    torch.cuda.synchronize()  # the primary context is current on this thread
    assert cu.cuModuleLoadData(C.byref(mod), image) == 0
    assert cu.cuModuleGetFunction(C.byref(fn), mod, b"module_put") == 0
    lib.nvshmemx_cumodule_init.argtypes = [C.c_void_p]
    lib.nvshmemx_cumodule_finalize.argtypes = [C.c_void_p]
    assert lib.nvshmemx_cumodule_init(mod) == 0
    count = 1000
    dst, src = nv.tensor((count,), torch.int32, zero=True), nv.tensor((count,), torch.int32)
    sig = nv.tensor((1,), torch.int64, zero=True)
    facts = torch.zeros(2, dtype=torch.int32, device="cuda")
    src.copy_(torch.arange(count, device="cuda", dtype=torch.int32) + 1000 * me)
    nv.barrier_all()
    torch.cuda.synchronize()
    right, left = (me + 1) % n, (me - 1) % n
    args = [C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), C.c_int(count), C.c_void_p(sig.data_ptr()), C.c_int(right), C.c_void_p(facts.data_ptr())]
    argv = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert cu.cuLaunchKernel(fn, 1, 1, 1, 256, 1, 1, 0, stream, argv, None) == 0
    nv.signal_wait(sig, count, nv.ComparisonType.CMP_EQ)   # the left neighbour's data has landed
    torch.cuda.synchronize()
    assert facts.tolist() == [me, n]
    assert torch.equal(dst.cpu(), torch.arange(count, dtype=torch.int32) + 1000 * left)
    assert nv.error_bits() == 0
    nv.barrier_all()
    assert lib.nvshmemx_cumodule_finalize(mod) == 0 and lib.nvshmemx_cumodule_finalize(mod) != 0
    assert cu.cuModuleUnload(mod) == 0
    for t in (dst, src, sig):
        nv.free_tensor(t)
    teardown(nv)


@worker
def rank_leaves_between_steps():
    """Failure detection without faulting a GPU: after a clean step one rank leaves (finalises nothing
    collectively, just stops taking part).  The others learn it on the host through the store before
    their next launch and stop too; a wait that would have depended on the missing rank is never issued."""
    nv = setup()
    n = WORLD
    x = nv.tensor((1024,), torch.float32)
    y = nv.tensor((1024,), torch.float32)
    x.fill_(1.0)
    nv.barrier_all()
    nv.reduce(0, y, x, "sum")
    torch.cuda.synchronize() if GPU else None
    assert float(y[0]) == n
    store = dist.distributed_c10d._get_default_store()
    dist.barrier()
    if RANK == n - 1:
        store.set("leaving", str(RANK))
    else:
        store.wait(["leaving"])
        gone = int(store.get("leaving"))
        assert gone == n - 1
        # no kernel that waits on the departed rank is launched; local work still runs
        y.mul_(2.0)
        torch.cuda.synchronize() if GPU else None
        assert float(y[0]) == 2 * n
    # Everyone is still alive here (leaving = no longer computing), so the collective shutdown is safe.
    teardown(nv)


def _leave_multicast():
    """Detaches this rank from every NVLink multicast object without any collective step."""
    try:
        from nvshmem_b200.bindings import host as H
        H.load().nvshmemx_b200_release_multicast()
    except Exception:
        pass


def _on_sigterm(signum, frame):
    raise SystemExit(143)


if __name__ == "__main__":
    import signal
    import traceback
    signal.signal(signal.SIGTERM, _on_sigterm)
    name = sys.argv[1]
    try:
        WORKERS[name]()
    except BaseException:
        # A rank that fails must not vanish while its memory is bound to a multicast object that the other
        # ranks' GPUs still use: unbind first (local calls only), then let the interpreter exit.
        traceback.print_exc()
        sys.stdout.flush()
        _leave_multicast()
        os._exit(1)
    print(f"rank {RANK}: {name} ok", flush=True)
