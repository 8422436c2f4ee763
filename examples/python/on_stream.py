"""Work ordered on a stream from Python: a local reduction, an all-reduce of the partial sums, and a correction that
depends on the global sum, with no host synchronisation between them (the Python form of examples/on-stream.cu).

  torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/python/on_stream.py
  NVSHMEM_HEAP_BACKEND=HOST torchrun --nproc-per-node 3 --master-addr 127.0.0.1 examples/python/on_stream.py   # no GPU

(Counterpart of the reference's nvshmem4py/examples/on-stream.py, whose local kernels are Numba kernels; here they are
torch operations on symmetric tensors, which run on the same stream as the collective.)
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem.core as nv  # noqa: E402

THRESHOLD, CORRECTION, NELEMS = 42, 7, 512


def main() -> int:
    gpu = torch.cuda.is_available() and os.environ.get("NVSHMEM_HEAP_BACKEND", "").upper() != "HOST"
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if gpu:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group("gloo")
    nv.init(device=local_rank if gpu else None, initializer_method="torch")
    me, n = nv.my_pe(), nv.n_pes()
    stream = torch.cuda.current_stream() if gpu else None

    data = nv.tensor((NELEMS,), torch.int64)
    partial = nv.tensor((1,), torch.int64)
    full = nv.tensor((1,), torch.int64)
    data.fill_(1)                                             # every element 1: the partial sum is NELEMS
    partial.copy_(data.sum().reshape(1))                      # "accumulate": on the current stream
    nv.reduce(nv.Teams.TEAM_WORLD, full, partial, "sum", stream=stream)
    over = full > THRESHOLD                                   # stays on the device: no host read before the correction
    data.sub_(over.to(torch.int64) * CORRECTION)              # "correct_accumulate"
    partial.copy_(data.sum().reshape(1))
    if gpu:
        torch.cuda.synchronize()
    want_full = n * NELEMS
    want_partial = NELEMS * (1 - CORRECTION) if want_full > THRESHOLD else NELEMS
    ok = int(full[0]) == want_full and int(partial[0]) == want_partial
    print(f"[{me} of {n}] run complete: full sum {int(full[0])}, corrected partial sum {int(partial[0])} {'ok' if ok else 'WRONG'}", flush=True)
    for t in (data, partial, full):
        nv.free_tensor(t)
    nv.finalize()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
