"""Triton kernels that communicate by themselves: one-sided stores into the neighbour's tensor, a fence, a signal, a
bounded wait for the own signal, and a sum computed inside the NVSwitch, all from inside the kernel with the helpers
of ``nvshmem.core.device.triton``.

  torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/triton_device_api.py

(Counterpart of the reference's nvshmem4py/examples/simple_p2p_kernel.py and device_custom_kernel.py, whose device
code is Numba.)  One kernel runs per GPU, so the kernels that wait for one another run on different GPUs.
"""
import os
import sys

import torch
import torch.distributed as dist
import triton
import triton.language as tl

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem.core as nv  # noqa: E402
from nvshmem.core.device import triton as nvt  # noqa: E402


@triton.jit
def ring_kernel(inbox_peer, sig_peer, sig_local, src, status, n, programs, BLOCK: tl.constexpr):
    """Every program stores its block into the neighbour's inbox, makes it visible and counts itself in on the
    neighbour's signal; program 0 then waits (bounded) until all programs of the other neighbour have counted in here."""
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    tl.store(inbox_peer + offs, tl.load(src + offs, mask=mask), mask=mask)
    tl.debug_barrier()          # all threads of the program have issued their stores
    nvt.fence()
    nvt.signal_add(sig_peer, 1)
    if pid == 0:
        ok = nvt.signal_wait_until_ge(sig_local, programs, 20000000)
        tl.store(status, ok)


@triton.jit
def switch_sum_kernel(mc_src, out, BLOCK4: tl.constexpr):
    """out[4 i .. 4 i + 3] = sum over all PEs of the same four floats, added by the switch."""
    i = tl.program_id(0)
    a, b, c, d = nvt.multimem_ld_reduce_add_f32x4(mc_src + 4 * i)
    tl.store(out + 4 * i + 0, a)
    tl.store(out + 4 * i + 1, b)
    tl.store(out + 4 * i + 2, c)
    tl.store(out + 4 * i + 3, d)


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.init(device=local_rank, initializer_method="torch")
    me, n = nv.my_pe(), nv.n_pes()
    stream = torch.cuda.current_stream()
    count, BLOCK = 8192, 1024
    programs = triton.cdiv(count, BLOCK)
    right, left = (me + 1) % n, (me - 1) % n

    inbox = nv.tensor((count,), torch.float32, zero=True)
    signal = nv.tensor((1,), torch.int64, zero=True)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mine = torch.arange(count, device="cuda", dtype=torch.float32) + 1000.0 * me
    peer_inbox, peer_signal = nv.get_peer_tensor(inbox, right), nv.get_peer_tensor(signal, right)
    nv.barrier_all(stream=stream)
    ring_kernel[(programs,)](peer_inbox, peer_signal, signal, mine, status, count, programs, BLOCK=BLOCK)
    torch.cuda.synchronize()
    ok = int(status[0]) == 1 and int(signal[0]) == programs
    ok = ok and torch.equal(inbox, torch.arange(count, device="cuda", dtype=torch.float32) + 1000.0 * left)

    have_mc = nv.heap_info()["mc_base"] != 0
    if have_mc:
        vals = nv.tensor((1024,), torch.float32)
        vals.copy_(torch.arange(1024, device="cuda", dtype=torch.float32) * (me + 1))
        out = torch.zeros(1024, dtype=torch.float32, device="cuda")
        mc_vals = nv.get_multicast_tensor(nv.Teams.TEAM_WORLD, vals)
        nv.barrier_all(stream=stream)
        switch_sum_kernel[(256,)](mc_vals, out, BLOCK4=4)
        nv.barrier_all(stream=stream)
        torch.cuda.synchronize()
        ok = ok and torch.equal(out, torch.arange(1024, device="cuda", dtype=torch.float32) * (n * (n + 1) // 2))
        nv.free_tensor(mc_vals)
        nv.free_tensor(vals)
    for t in (peer_inbox, peer_signal, inbox, signal):
        nv.free_tensor(t)
    print(f"PE {me} of {n}: {'ok' if ok else 'WRONG'} (in-switch sum {'ran' if have_mc else 'skipped: no NVLS'})", flush=True)
    nv.finalize()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
