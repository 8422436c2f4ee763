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


@pytest.mark.parametrize("G,N,K,act", [(4, 256, 128, None), (7, 512, 320, None), (5, 512, 256, "swiglu"), (32, 1024, 512, "swiglu")])
def test_grouped_gemm_over_ragged_groups(G, N, K, act):
    """Rows fall into groups of uneven size (some empty, none a multiple of 128); each group has its own weight.
    The group boundaries are read by the kernel from device memory."""
    from nvshmem_b200.ops import fused_gemm as fg
    torch.manual_seed(G * 1000 + N + K)
    sizes = torch.randint(0, 400, (G,))
    sizes[G // 2] = 0                      # an empty group in the middle
    sizes[0] = 129                         # one full block and a block of one row
    offs = torch.zeros(G + 1, dtype=torch.int32)
    offs[1:] = sizes.cumsum(0).to(torch.int32)
    rows = int(offs[-1])
    cap = rows + 77                        # the buffers are larger than what the groups use
    x = torch.randn(cap, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(G, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    out_cols = N // 2 if act == "swiglu" else N
    out = torch.full((cap, out_cols), 7.0, dtype=torch.bfloat16, device="cuda")
    w_used = fg.interleave_gate_up(w) if act == "swiglu" else w
    fg.grouped_gemm(x, w_used, offs.cuda(), out=out, act=act)
    torch.cuda.synchronize()
    fg.check_errors()
    assert bool((out[rows:] == 7.0).all()), "rows beyond the last group were written"
    for g in range(G):
        lo, hi = int(offs[g]), int(offs[g + 1])
        if hi == lo:
            continue
        ref = x[lo:hi].float() @ w[g].float().t()
        if act == "swiglu":
            ref = torch.nn.functional.silu(ref[:, :N // 2]) * ref[:, N // 2:]
        err = (out[lo:hi].float() - ref).abs().max().item()
        assert err <= ref.abs().max().item() * 2 ** -6 + 2e-3, (g, lo, hi, err)


def test_interleave_gate_up_orders_rows_in_blocks_of_32():
    from nvshmem_b200.ops import fused_gemm as fg
    F, K = 64, 4
    w = torch.arange(2 * F, dtype=torch.float32).view(2 * F, 1).expand(2 * F, K).contiguous()
    r = fg.interleave_gate_up(w)[:, 0].tolist()
    assert r[:32] == list(range(0, 32)) and r[32:64] == list(range(F, F + 32)) and r[64:96] == list(range(32, 64)) and r[96:] == list(range(F + 32, 2 * F))
