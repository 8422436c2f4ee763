"""Triton kernels on symmetric memory: a kernel that writes straight into a peer's tensor over NVLink, and a kernel
that stores through the NVLink-multicast alias of a tensor (one `multimem.st` per element reaches every PE).

  torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/triton_interop.py

The library supplies the memory (symmetric tensors, their peer and multicast views) and the ordering (barriers on
the stream); the kernels are ordinary Triton.  (counterpart of the reference's
nvshmem4py/examples/triton_comm_kernels.py and torch_triton_interop.py)
"""
import os
import sys

import torch
import torch.distributed as dist
import triton
import triton.language as tl

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem_b200.core as nv  # noqa: E402


@triton.jit
def put_kernel(dst_ptr, src_ptr, n, BLOCK: tl.constexpr):
    """dst (a peer's memory, mapped into this process) = src."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    tl.store(dst_ptr + offs, tl.load(src_ptr + offs, mask=mask), mask=mask)


@triton.jit
def multicast_store_kernel(mc_ptr, src_ptr, n, BLOCK: tl.constexpr):
    """Stores src (int64 elements) through the multicast address: the switch delivers every element to all PEs."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    v = tl.load(src_ptr + offs, mask=mask, other=0)
    addr = (mc_ptr + offs).to(tl.int64, bitcast=True)
    safe = tl.where(mask, addr, (mc_ptr + 0).to(tl.int64, bitcast=True))  # masked lanes rewrite element 0 with its own value below
    val = tl.where(mask, v, tl.load(src_ptr))
    tl.inline_asm_elementwise("multimem.st.relaxed.sys.global.u64 [$1], $2; mov.u32 $0, 0;", "=r,l,l", [safe, val], dtype=tl.int32, is_pure=False, pack=1)


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.init(device=local_rank, initializer_method="torch")
    me, n = nv.my_pe(), nv.n_pes()
    stream = torch.cuda.current_stream()
    count, BLOCK = 10000, 1024
    grid = (triton.cdiv(count, BLOCK),)
    ok = True

    # 1. every PE writes its pattern into the inbox of its right-hand neighbour with a Triton kernel
    inbox = nv.tensor((count,), torch.float32, zero=True)
    mine = torch.arange(count, device="cuda", dtype=torch.float32) + 1000.0 * me
    right, left = (me + 1) % n, (me - 1) % n
    peer_inbox = nv.get_peer_tensor(inbox, right)
    nv.barrier_all(stream=stream)
    put_kernel[grid](peer_inbox, mine, count, BLOCK=BLOCK)
    nv.barrier_all(stream=stream)          # completes the stores of all PEs
    torch.cuda.synchronize()
    ok = ok and torch.equal(inbox, torch.arange(count, device="cuda", dtype=torch.float32) + 1000.0 * left)

    # 2. PE 0 broadcasts a table through the multicast alias; without NVLS the step is skipped
    table = nv.tensor((count,), torch.int64, zero=True)
    have_mc = nv.heap_info()["mc_base"] != 0
    if have_mc:
        mc_table = nv.get_multicast_tensor(nv.Teams.TEAM_WORLD, table)
        src = torch.arange(count, device="cuda", dtype=torch.int64) * 3 + 7
        nv.barrier_all(stream=stream)
        if me == 0:
            multicast_store_kernel[grid](mc_table, src, count, BLOCK=BLOCK)
        nv.barrier_all(stream=stream)
        torch.cuda.synchronize()
        ok = ok and torch.equal(table, src)
        nv.free_tensor(mc_table)
    nv.free_tensor(peer_inbox)
    print(f"PE {me} of {n}: {'ok' if ok else 'WRONG'} (multicast step {'ran' if have_mc else 'skipped: no NVLS'})")
    for t in (inbox, table):
        nv.free_tensor(t)
    nv.finalize()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
