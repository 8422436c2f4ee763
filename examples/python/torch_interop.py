"""Symmetric torch tensors, on-stream collectives and one-sided transfers from Python.

  torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/python/torch_interop.py

(counterpart of the reference's nvshmem4py/examples/torch_triton_interop.py; the device side there is a
Triton kernel, here the library's own kernels)
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem_b200.core as nv  # noqa: E402


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.init(device=local_rank, initializer_method="torch")  # the 128-byte unique id travels over torch.distributed once
    me, n = nv.my_pe(), nv.n_pes()
    stream = torch.cuda.current_stream()

    # all-reduce of a symmetric tensor, ordered on the current stream
    x = nv.tensor((1 << 20,), torch.float32)
    y = nv.tensor((1 << 20,), torch.float32)
    x.fill_(float(me + 1))
    nv.barrier_all(stream=stream)
    nv.reduce(nv.Teams.TEAM_WORLD, y, x, "sum", stream=stream)
    torch.cuda.synchronize()
    ok = bool((y == n * (n + 1) / 2).all())

    # one-sided: write my rank into my slot of the right-hand neighbour's table, then tell it
    table = nv.tensor((n,), torch.int64, zero=True)
    mine = nv.tensor((1,), torch.int64)
    signal = nv.tensor((1,), torch.int64, zero=True)
    mine.fill_(me)
    nv.barrier_all(stream=stream)
    right = (me + 1) % n
    nv.put_signal(table[me:me + 1], mine, signal, 1, nv.SignalOp.SIGNAL_ADD, right, stream=stream)
    nv.signal_wait(signal, 1, nv.ComparisonType.CMP_GE, stream=stream)
    torch.cuda.synchronize()
    left = (me + n - 1) % n
    ok = ok and int(table[left]) == left

    # the same memory through a peer mapping (plain loads over NVLink) and through the multicast alias
    peer_view = nv.get_peer_tensor(x, right)
    ok = ok and float(peer_view[0]) == float(right + 1)
    print(f"PE {me} of {n}: {'ok' if ok else 'WRONG'}; heap {nv.heap_info()}")
    for t in (x, y, table, mine, signal):
        nv.free_tensor(t)
    nv.finalize()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
