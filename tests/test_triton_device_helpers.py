"""The Triton device helpers (nvshmem.core.device.triton) compile for sm_100 with no GPU present: Triton lowers a
kernel that uses every helper to PTX and ptxas assembles it, which checks the inline instructions (fence, multimem
store / load-reduce / reduction) and the release / acquire atomics.  Behaviour is tested on GPUs by the example
examples/python/triton_device_api.py."""
import sys
import textwrap

import pytest

triton = pytest.importorskip("triton")


def test_every_helper_compiles_for_sm_100(tmp_path, monkeypatch):
    from triton.backends.compiler import GPUTarget
    from triton.compiler import ASTSource
    (tmp_path / "uses_helpers.py").write_text(textwrap.dedent('''
        import triton
        import triton.language as tl
        from nvshmem.core.device import triton as nvt

        @triton.jit
        def kernel(inbox_peer, sig_peer, sig_local, out, src, mc, n, BLOCK: tl.constexpr):
            pid = tl.program_id(0)
            offs = pid * BLOCK + tl.arange(0, BLOCK)
            mask = offs < n
            tl.store(inbox_peer + offs, tl.load(src + offs, mask=mask), mask=mask)
            nvt.fence()
            nvt.signal_add(sig_peer, 1)
            if pid == 0:
                nvt.signal_set(sig_peer + 1, 9)
                ok = nvt.signal_wait_until_ge(sig_local, 1, 1000)
                tl.store(out, ok)
                tl.store(out + 1, nvt.signal_load(sig_local).to(tl.int32))
                a, b, c, d = nvt.multimem_ld_reduce_add_f32x4(mc)
                nvt.multimem_st_f32x4(mc + 4, a, b, c, d)
                nvt.multimem_red_add_f32(mc + 8, a)
                nvt.multimem_st_u64((mc + 16).to(tl.pointer_type(tl.int64)), tl.full((), 5, tl.int64))
    '''))
    monkeypatch.syspath_prepend(str(tmp_path))
    import uses_helpers
    sig = {"inbox_peer": "*fp32", "sig_peer": "*i64", "sig_local": "*i64", "out": "*i32", "src": "*fp32", "mc": "*fp32", "n": "i32", "BLOCK": "constexpr"}
    try:
        compiled = triton.compile(ASTSource(fn=uses_helpers.kernel, signature=sig, constexprs={"BLOCK": 256}), target=GPUTarget("cuda", 100, 32))
    except Exception as e:  # a Triton build that cannot compile without a device
        if "device" in str(e).lower() or "driver" in str(e).lower():
            pytest.skip(f"this Triton cannot compile offline: {e}")
        raise
    ptx = compiled.asm["ptx"]
    for needle in ("fence.acq_rel.sys", "multimem.ld_reduce.relaxed.sys.global.add.v4.f32", "multimem.st.relaxed.sys.global.v4.f32",
                   "multimem.st.relaxed.sys.global.u64", "multimem.red.relaxed.sys.global.add.f32"):
        assert needle in ptx, needle
    lines = ptx.splitlines()
    assert any("acquire" in l and ".sys" in l for l in lines), "the signal polls must be system-scope acquires"
    assert any("release" in l and ".sys" in l for l in lines), "the signal updates must be system-scope releases"
    assert len(compiled.asm.get("cubin", b"")) > 0
    sys.modules.pop("uses_helpers", None)


def test_numba_bindings_say_what_to_use_instead():
    import nvshmem.core.device as dev
    with pytest.raises(ImportError, match="triton"):
        dev.numba
