"""Memory that the application allocates itself (CUDA virtual memory management) becomes symmetric.

  torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/external_memory.py

Each rank creates one 512 MB physical allocation with cuMemCreate (shareable as a POSIX file descriptor),
maps it, and registers it: the library maps every rank's allocation into every rank's view of the heap and
returns the symmetric address, which then works with all RMA and collective calls.
(counterpart of the reference's nvshmem4py/examples/torch_mempool.py, which reaches the same registration
call through a torch pluggable allocator)
"""
import os
import sys

import torch
import torch.distributed as dist
from cuda.bindings import driver as cu

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import nvshmem_b200.core as nv  # noqa: E402

BYTES = 512 << 20  # a multiple of the heap's growth granule


def check(result):
    err = result[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return result[1] if len(result) == 2 else result[1:]


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.init(device=local_rank, initializer_method="torch")
    me, n = nv.my_pe(), nv.n_pes()

    prop = cu.CUmemAllocationProp()
    prop.type = cu.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
    prop.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    prop.location.id = local_rank
    prop.requestedHandleTypes = cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
    handle = check(cu.cuMemCreate(BYTES, prop, 0))
    va = check(cu.cuMemAddressReserve(BYTES, 0, 0, 0))
    check(cu.cuMemMap(va, BYTES, 0, handle, 0))
    access = cu.CUmemAccessDesc()
    access.location = prop.location
    access.flags = cu.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
    check(cu.cuMemSetAccess(va, BYTES, [access], 1))

    sym = nv.register_external_buffer(int(va), BYTES)            # collective
    words = torch.as_tensor(sym, device=f"cuda:{local_rank}").view(torch.float32)
    src, dst = words[:4096], words[4096:8192]
    src.fill_(float(me))
    dst.zero_()
    stream = torch.cuda.current_stream()
    nv.barrier_all(stream=stream)
    nv.put(dst, src, (me + 1) % n, stream=stream)                # both sides live in the registered memory
    nv.barrier_all(stream=stream)
    torch.cuda.synchronize()
    ok = bool((dst == float((me + n - 1) % n)).all())
    print(f"PE {me}: put through registered memory {'ok' if ok else 'WRONG'}")

    del words, src, dst
    nv.unregister_external_buffer(sym)                           # collective
    check(cu.cuMemUnmap(va, BYTES))
    check(cu.cuMemAddressFree(va, BYTES))
    check(cu.cuMemRelease(handle))
    nv.finalize()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
