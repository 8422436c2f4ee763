"""``@triton.jit`` helpers for kernels that communicate through symmetric memory.

A Triton kernel gets at a peer's memory through an ordinary pointer: ``nvshmem.core.get_peer_tensor(t, pe)`` is PE
``pe``'s copy of the symmetric tensor ``t`` mapped into this process, and ``get_multicast_tensor(team, t)`` is its
NVLink-multicast alias.  Loads and stores on those tensors are one-sided gets and puts; what a kernel needs beyond
that is ordering, signalling and the multicast instructions, which is what this module adds:

=====================================  =====================================================================
``fence()``                            orders this thread's earlier memory operations before its later ones for
                                       every observer (``fence.acq_rel.sys``; the device ``nvshmem_fence``)
``signal_set(sig, value)``             release-store of a 64-bit signal word (peer or local)
``signal_add(sig, value)``             release-add (``NVSHMEM_SIGNAL_ADD``)
``signal_load(sig)``                   acquire-load of a signal word
``signal_wait_until_ge(sig, v, n)``    polls (acquire) at most ``n`` times; 1 when the word reached ``v``, else 0:
                                       a wait never hangs the GPU, the kernel decides what to do when it runs out
``multimem_st_u64 / _f32x4``           store through a multicast address: the switch delivers to every PE
``multimem_ld_reduce_add_f32x4``       load through a multicast address: the switch returns the sum over all PEs
``multimem_red_add_f32``               reduction into every PE's copy
=====================================  =====================================================================

All take scalar pointers (one element per program); vectorised use goes through ordinary ``tl.load`` / ``tl.store`` on
the peer view.  The multicast helpers need a GPU and a heap with a multicast window (``heap_info()["mc_base"] != 0``).
(reference counterpart: nvshmem4py/nvshmem/core/device/numba/{rma,amo,direct}.py and the inline ``multimem.st`` of
nvshmem4py/examples/triton_comm_kernels.py)
"""
import triton
import triton.language as tl


@triton.jit
def fence():
    zero = tl.full((), 0, tl.int32)
    tl.inline_asm_elementwise("fence.acq_rel.sys; mov.u32 $0, $1;", "=r,r", [zero], dtype=tl.int32, is_pure=False, pack=1)


@triton.jit
def signal_set(sig_ptr, value):
    tl.atomic_xchg(sig_ptr, value, sem="release", scope="sys")


@triton.jit
def signal_add(sig_ptr, value):
    tl.atomic_add(sig_ptr, value, sem="release", scope="sys")


@triton.jit
def signal_load(sig_ptr):
    return tl.atomic_add(sig_ptr, 0, sem="acquire", scope="sys")


@triton.jit
def signal_wait_until_ge(sig_ptr, value, max_polls):
    ok = tl.full((), 0, tl.int32)
    polls = tl.full((), 0, tl.int32)
    while (ok == 0) & (polls < max_polls):
        seen = tl.atomic_add(sig_ptr, 0, sem="acquire", scope="sys")
        ok = (seen >= value).to(tl.int32)
        polls += 1
    return ok


@triton.jit
def multimem_st_u64(mc_ptr, value):
    addr = mc_ptr.to(tl.int64, bitcast=True)
    tl.inline_asm_elementwise("multimem.st.relaxed.sys.global.u64 [$1], $2; mov.u32 $0, 0;", "=r,l,l", [addr, value], dtype=tl.int32, is_pure=False, pack=1)


@triton.jit
def multimem_st_f32x4(mc_ptr, a, b, c, d):
    """Four consecutive floats at a 16-byte aligned multicast address."""
    addr = mc_ptr.to(tl.int64, bitcast=True)
    tl.inline_asm_elementwise("multimem.st.relaxed.sys.global.v4.f32 [$1], {$2, $3, $4, $5}; mov.u32 $0, 0;", "=r,l,f,f,f,f", [addr, a, b, c, d], dtype=tl.int32,
                              is_pure=False, pack=1)


@triton.jit
def multimem_ld_reduce_add_f32x4(mc_ptr):
    """Sum over all PEs of four consecutive floats at a 16-byte aligned multicast address (computed in the switch)."""
    addr = mc_ptr.to(tl.int64, bitcast=True)
    return tl.inline_asm_elementwise("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {$0, $1, $2, $3}, [$4];", "=f,=f,=f,=f,l", [addr],
                                     dtype=(tl.float32, tl.float32, tl.float32, tl.float32), is_pure=False, pack=1)


@triton.jit
def multimem_red_add_f32(mc_ptr, value):
    addr = mc_ptr.to(tl.int64, bitcast=True)
    tl.inline_asm_elementwise("multimem.red.relaxed.sys.global.add.f32 [$1], $2; mov.u32 $0, 0;", "=r,l,f", [addr, value], dtype=tl.int32, is_pure=False, pack=1)
