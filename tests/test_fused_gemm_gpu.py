"""Numerics of the tcgen05 GEMM kernel against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, w):
    return x.float() @ w.float().t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 192), (1024, 768, 512), (2048, 256, 3584), (384, 1280, 1088)])
def test_gemm_matches_fp32_reference(M, N, K):
    from nvshmem_b200.ops import fused_gemm as fg
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    out = fg.gemm(x, w)
    torch.cuda.synchronize()
    fg.check_errors()
    ref = _ref(x, w)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    # bf16 output rounding: half an ulp of the largest magnitude, plus accumulation-order slack
    assert err <= scale * 2 ** -7 + 1e-3, f"max abs err {err} at scale {scale}"


def test_gemm_structured_operands_catch_layout_errors():
    """Operands with distinct values per row and per k make a wrong swizzle or descriptor visible."""
    from nvshmem_b200.ops import fused_gemm as fg
    M, N, K = 256, 256, 128
    x = torch.zeros(M, K, device="cuda")
    w = torch.zeros(N, K, device="cuda")
    x[torch.arange(M), torch.arange(M) % K] = 1.0          # row i picks column i % K of w^T
    w += (torch.arange(N, device="cuda").float()[:, None] % 7 + 1) * (torch.arange(K, device="cuda").float()[None, :] % 5 + 1)
    out = fg.gemm(x.to(torch.bfloat16), w.to(torch.bfloat16))
    torch.cuda.synchronize()
    ref = _ref(x.to(torch.bfloat16), w.to(torch.bfloat16))
    assert torch.equal(out.float(), ref.to(torch.bfloat16).float())


def test_gemm_rejects_bad_shapes():
    from nvshmem_b200.ops import fused_gemm as fg
    x = torch.zeros(100, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(fg.FusedGemmError):
        fg.gemm(x, w)


def test_gemm_with_few_ctas_walks_all_tiles():
    from nvshmem_b200.ops import fused_gemm as fg
    torch.manual_seed(5)
    x = torch.randn(1024, 320, device="cuda").to(torch.bfloat16)
    w = torch.randn(1024, 320, device="cuda").to(torch.bfloat16)
    out = fg.gemm(x, w, max_ctas=3)  # 32 tiles on 3 CTAs: exercises the persistent loop and both TMEM buffers
    torch.cuda.synchronize()
    ref = _ref(x, w)
    assert (out.float() - ref).abs().max().item() <= ref.abs().max().item() * 2 ** -7 + 1e-3
