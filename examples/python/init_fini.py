"""Ways to start and stop the library from Python, one after the other in the same processes.

  torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/python/init_fini.py          # GPUs
  NVSHMEM_HEAP_BACKEND=HOST torchrun --nproc-per-node 3 --master-addr 127.0.0.1 examples/python/init_fini.py   # no GPU

1. unique id made by rank 0 and broadcast in place as bytes (``uid._data.view(numpy.int8)``), then ``init(uid=...)``;
2. the same through ``broadcast_object_list``;
3. ``initializer_method="torch"`` (the layer fetches and distributes the id itself);
4. the pointer-level bindings (``nvshmem.bindings``): attribute structs and ``hostlib_init_attr``.

Each round allocates, runs a barrier and finalises.  (Counterpart of the reference's
nvshmem4py/examples/init_fini.py, whose launchers are mpi4py and torchrun; there is no MPI here.)
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem.core as nv  # noqa: E402  (the reference package's import name; the same module as nvshmem_b200.core)
import nvshmem.bindings as bindings  # noqa: E402


def main() -> int:
    gpu = torch.cuda.is_available() and os.environ.get("NVSHMEM_HEAP_BACKEND", "").upper() != "HOST"
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if gpu:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group("gloo")
    rank, nranks = dist.get_rank(), dist.get_world_size()
    device = local_rank if gpu else None
    where = torch.device("cuda", local_rank) if gpu else torch.device("cpu")

    def use_it():
        x = nv.tensor((16,), torch.float32)
        x.fill_(rank)
        nv.barrier_all()
        ok = nv.my_pe() == rank and nv.n_pes() == nranks
        nv.free_tensor(x)
        nv.finalize()
        return ok

    ok = True
    # 1. in-place broadcast of the id's bytes
    uid = nv.get_unique_id(empty=rank != 0)
    raw = torch.from_numpy(uid._data.view(np.int8)).to(where)
    dist.broadcast(raw, src=0)
    uid._data.view(np.int8)[:] = raw.cpu().numpy()
    nv.init(device=device, uid=uid, rank=rank, nranks=nranks, initializer_method="uid")
    ok &= use_it()
    # 2. the id as a Python object
    box = [nv.get_unique_id().to_bytes() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    nv.init(device=device, uid=box[0], rank=rank, nranks=nranks)
    ok &= use_it()
    # 3. the layer does it
    nv.init(device=device, initializer_method="torch")
    ok &= use_it()
    # 4. pointer-level bindings
    uid4 = bindings.UniqueId()
    if rank == 0:
        bindings.get_uniqueid(uid4.ptr)
    raw = torch.from_numpy(uid4._data.view(np.int8)).to(where)
    dist.broadcast(raw, src=0)
    uid4._data.view(np.int8)[:] = raw.cpu().numpy()
    attr = bindings.InitAttr()
    bindings.set_attr_uniqueid_args(rank, nranks, uid4.ptr, attr.ptr)
    bindings.hostlib_init_attr(bindings.Flags.INIT_WITH_UNIQUEID, attr.ptr)
    p = bindings.malloc(1024)
    bindings.barrier_all()
    ok &= p != 0 and bindings.my_pe() == rank and bindings.team_n_pes(bindings.Team_id.TEAM_WORLD) == nranks
    bindings.free(p)
    bindings.hostlib_finalize()
    print(f"PE {rank} of {nranks}: four start-ups and shut-downs {'ok' if ok else 'WRONG'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
