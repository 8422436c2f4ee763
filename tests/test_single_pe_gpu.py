"""One PE on one GPU: VMM heap, symmetric tensors, host RMA to self, collectives of size one, fused ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nv():
    import nvshmem_b200.core as nv
    torch.cuda.set_device(0)
    nv.init(device=0, uid=nv.get_unique_id(), rank=0, nranks=1)
    yield nv
    nv.finalize()


def test_world_of_one(nv):
    assert nv.my_pe() == 0 and nv.n_pes() == 1
    info = nv.heap_info()
    assert info["backed"] >= 1 << 30 and info["stride"] >= info["backed"]
    assert "B200" in nv.topology() or "NVIDIA" in nv.topology()


def test_tensor_alloc_put_get_roundtrip(nv):
    a = nv.tensor((1 << 20,), torch.float32)
    b = nv.tensor((1 << 20,), torch.float32)
    src = torch.rand(1 << 20, device="cuda")
    nv.put(a, src, 0)
    nv.get(b, a, 0)
    nv.quiet()
    torch.cuda.synchronize()
    assert torch.equal(b, src)
    nv.free_tensor(a)
    nv.free_tensor(b)


def test_heap_growth_keeps_old_data(nv):
    small = nv.tensor((1024,), torch.int32)
    small.copy_(torch.arange(1024, dtype=torch.int32, device="cuda"))
    before = nv.heap_info()["chunks"]
    big = nv.tensor(((3 << 30) // 4,), torch.float32)  # larger than the initial 1 GiB: forces growth
    assert nv.heap_info()["chunks"] > before
    big[-1] = 7.0
    torch.cuda.synchronize()
    assert torch.equal(small.cpu(), torch.arange(1024, dtype=torch.int32))
    assert float(big[-1]) == 7.0
    nv.free_tensor(big)
    nv.free_tensor(small)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32, torch.int64])
def test_collectives_on_one_pe_are_copies(nv, dtype):
    n = 4096
    src = nv.tensor((n,), dtype)
    dst = nv.tensor((n,), dtype)
    src.copy_((torch.arange(n, device="cuda") % 97).to(dtype))
    for coll in ("reduce", "reducescatter", "fcollect", "alltoall", "broadcast"):
        dst.zero_()
        nv.collective_on_buffer(coll, 0, dst, src, op="sum")
        nv.barrier_all()
        torch.cuda.synchronize()
        assert torch.equal(dst, src), coll
    assert nv.error_bits() == 0
    nv.free_tensor(src)
    nv.free_tensor(dst)


def test_signal_and_wait_on_stream(nv):
    sig = nv.tensor((1,), torch.int64, zero=True)
    nv.signal_op(sig, 5, nv.SignalOp.SIGNAL_SET, 0)
    nv.signal_wait(sig, 5, nv.ComparisonType.CMP_GE)
    nv.signal_op(sig, 3, nv.SignalOp.SIGNAL_ADD, 0)
    torch.cuda.synchronize()
    assert nv.signal_fetch(sig) == 8
    nv.free_tensor(sig)


def test_bounded_wait_reports_timeout_instead_of_hanging(nv):
    """A signal that nobody sets: the wait kernel gives up after the bound and the status says so."""
    sig = nv.tensor((1,), torch.int64, zero=True)
    nv.set_wait_timeout_ms(200)
    nv.clear_errors()
    from nvshmem_b200.bindings import host as H
    # CMP_GT cannot use the stream memory operation, so this runs the device wait loop.
    nv.signal_wait(sig, 1, nv.ComparisonType.CMP_GT)
    torch.cuda.synchronize()
    assert nv.error_bits() & H.ERR_WAIT_TIMEOUT
    nv.clear_errors()
    nv.set_wait_timeout_ms(30000)
    nv.free_tensor(sig)


def test_fused_ops_single_pe(nv):
    from nvshmem_b200.ops import fused_gemm as fg
    torch.manual_seed(1)
    M, N, K = 512, 512, 256
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    tol = ref.abs().max().item() * 2 ** -7 + 1e-3
    rs = fg.GemmReduceScatter(M, N, mode="rs")
    assert (rs(x, w).float() - ref).abs().max().item() <= tol
    ar = fg.GemmReduceScatter(M, N, mode="ar")
    assert (ar(x, w).float() - ref).abs().max().item() <= tol
    ag = fg.AllGatherGemm(M, K)
    ag.shard.copy_(x)
    assert (ag(w).float() - ref).abs().max().item() <= tol
    fg.check_errors()


def test_tp_mlp_forward_backward_single_pe(nv):
    from nvshmem_b200.models.tp_mlp import TensorParallelMLP
    torch.manual_seed(2)
    mlp = TensorParallelMLP(hidden=512, ffn=1024, tokens=256)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = mlp(x)
    y.float().pow(2).mean().backward()
    ref = mlp.reference(x.detach())
    assert (y.float() - ref).abs().max().item() <= 0.03 * ref.abs().max().item() + 1e-2
    # gradient check against autograd through the fp32 reference
    x32 = x.detach().float().requires_grad_(True)
    w1 = mlp.up.weight.detach().float().requires_grad_(True)
    w2 = mlp.down.weight.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(x32 @ w1.t(), approximate="tanh") @ w2.t()
    yr.pow(2).mean().backward()
    for got, want in ((x.grad, x32.grad), (mlp.up.weight.grad, w1.grad), (mlp.down.weight.grad, w2.grad)):
        denom = want.abs().max().item() + 1e-12
        assert (got.float() - want).abs().max().item() / denom < 0.06


def test_moe_dispatch_combine_single_pe(nv):
    """All experts local: dispatch is a permutation by expert, combine its weighted inverse."""
    import tests.workers as W
    W._moe_check(nv, "bf16", T=200, H=512, K=4, E=16, seed=11)
    W._moe_check(nv, "fp8", T=128, H=1024, K=8, E=32, seed=12)


@pytest.mark.parametrize("payload,tol", [("bf16", 0.03), ("fp8", 0.08)])
def test_moe_block_matches_fp32_reference_single_pe(nv, payload, tol):
    """Router + dispatch + expert MLPs + combine against a plain PyTorch fp32 version of the same block."""
    from nvshmem_b200.models.moe_block import ExpertParallelMoE, reference_forward
    from nvshmem_b200.ops import fused_gemm as fg
    T, H, F, E, K = 192, 256, 384, 8, 2
    block = ExpertParallelMoE(T, H, F, E, K, payload=payload, seed=3, wait_limit_ms=5000)
    torch.manual_seed(17)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    got = block(x)
    torch.cuda.synchronize()
    fg.check_errors()
    want = reference_forward(x, block.router, block.w_in, block.w_out, K)
    err = (got.float() - want).abs().max().item()
    assert err <= tol * want.abs().max().item() + 1e-3, (payload, err, want.abs().max().item())
    block.close()


def test_copy_engine_collectives_on_one_pe(nv):
    """The copy-engine variants of fcollect / alltoall / broadcast (one memcpy per member + barrier)."""
    n = 1 << 16
    src = nv.tensor((n,), torch.float32)
    dst = nv.tensor((n,), torch.float32)
    src.copy_(torch.arange(n, device="cuda", dtype=torch.float32))
    nv.set_ce_collectives(1)
    try:
        for coll in ("fcollect", "alltoall", "broadcast"):
            dst.zero_()
            nv.collective_on_buffer(coll, 0, dst, src, op="sum")
            nv.barrier_all()
            torch.cuda.synchronize()
            assert torch.equal(dst, src), coll
    finally:
        nv.set_ce_collectives(0)
    assert nv.error_bits() == 0
    nv.free_tensor(src)
    nv.free_tensor(dst)


def test_device_code_in_a_separately_loaded_module():
    """A cubin built from tests/data/device_module_kernel.cu is loaded with the driver API, given the library state with
    nvshmemx_cumodule_init and puts to PE 0 (itself).  Runs as a child process with its own initialisation."""
    from tests._mp import run_workers
    run_workers("device_module_via_driver_api", 1, gpu=True, env={"NVSHMEM_DISABLE_NVLS": "1"}, timeout=300)
