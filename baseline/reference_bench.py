"""Reference arm of bench.py: the same metric on the same configuration with the UNMODIFIED reference
build in ``baseline/_ref`` (NVIDIA NVSHMEM, built from its own sources with its own CMake).

Per step and rank: cuBLAS bf16 GEMM (``torch.matmul``) writes the partial product into a buffer on the
reference's symmetric heap, then the reference library's own
``nvshmemx_bfloat16_sum_reducescatter_on_stream`` reduces and scatters it on the same stream.  The
end-to-end run is the same stack of tensor-parallel MLP blocks as the other arm's, built from the reference's
``nvshmemx_bfloat16_fcollect_on_stream`` (all-gather), cuBLAS GEMMs, torch's tanh-GELU and the reference's
reduce-scatter.  The library is driven through its public host API (unique-id init, ``nvshmem_malloc``, the
typed on-stream collectives) with ctypes; none of this repository's kernels, heap or Python layer is on that path.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


class _UniqueId(C.Structure):
    _fields_ = [("version", C.c_int), ("internal", C.c_char * 124)]


class _UidArgs(C.Structure):
    _fields_ = [("version", C.c_int), ("id", C.POINTER(_UniqueId)), ("myrank", C.c_int), ("nranks", C.c_int)]


class _InitArgs(C.Structure):
    _fields_ = [("version", C.c_int), ("uid_args", _UidArgs), ("cuda_device_id", C.c_int), ("content", C.c_char * 92)]


class _InitAttr(C.Structure):
    _fields_ = [("version", C.c_int), ("mpi_comm", C.c_void_p), ("args", _InitArgs)]


class _Sym:
    """A span of the reference's symmetric heap that torch can wrap (CUDA array interface)."""

    def __init__(self, ptr, nbytes):
        self.ptr, self.nbytes = ptr, nbytes

    @property
    def __cuda_array_interface__(self):
        return {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3, "strides": None}


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run(args, M, N, K_LOCAL) -> dict:
    lib_path = REF / "lib" / "libnvshmem_host.so"
    plugin = REF / "lib" / "nvshmem_bootstrap_uid.so"
    if not lib_path.exists() or not plugin.exists():
        return unavailable("baseline/_ref holds no reference build (the reference is a CMake project that pip cannot install; its CMake build was not found)")
    import torch
    import torch.distributed as dist
    from bench import ClockSampler, timed_runs  # shared timing harness

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    os.environ["NVSHMEM_BOOTSTRAP_UID_PLUGIN"] = str(plugin)
    os.environ.setdefault("NVSHMEM_SYMMETRIC_SIZE", "3G")
    os.environ.setdefault("NVSHMEM_BOOTSTRAP_UID_SOCK_IFNAME", "lo")
    lib = C.CDLL(str(lib_path), mode=C.RTLD_GLOBAL)
    lib.nvshmem_malloc.restype = C.c_void_p
    lib.nvshmem_malloc.argtypes = [C.c_size_t]
    lib.nvshmem_free.argtypes = [C.c_void_p]
    lib.nvshmemx_bfloat16_sum_reducescatter_on_stream.restype = C.c_int
    lib.nvshmemx_bfloat16_sum_reducescatter_on_stream.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.nvshmemx_bfloat16_fcollect_on_stream.restype = C.c_int
    lib.nvshmemx_bfloat16_fcollect_on_stream.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]

    uid = _UniqueId()
    uid.version = (1 << 16) + C.sizeof(_UniqueId)
    if rank == 0:
        st = lib.nvshmemx_get_uniqueid(C.byref(uid))
        if st != 0:
            return unavailable(f"reference nvshmemx_get_uniqueid returned {st}")
    if world > 1:
        payload = [bytes(C.string_at(C.addressof(uid), C.sizeof(uid))) if rank == 0 else None]
        dist.broadcast_object_list(payload, src=0)
        C.memmove(C.addressof(uid), payload[0], C.sizeof(uid))
    attr = _InitAttr()
    attr.version = (2 << 16) + C.sizeof(_InitAttr)
    attr.args.version = (2 << 16) + C.sizeof(_InitArgs)
    attr.args.uid_args.version = (1 << 16) + C.sizeof(_UidArgs)
    attr.args.cuda_device_id = -1
    lib.nvshmemx_set_attr_uniqueid_args(rank, world, C.byref(uid), C.byref(attr))
    st = lib.nvshmemx_hostlib_init_attr(8, C.byref(attr))  # NVSHMEMX_INIT_WITH_UNIQUEID
    if st != 0:
        return unavailable(f"reference nvshmemx_hostlib_init_attr returned {st}")

    rows = M // world
    partial_bytes, out_bytes = M * N * 2, rows * N * 2
    p_ptr, o_ptr = lib.nvshmem_malloc(partial_bytes), lib.nvshmem_malloc(out_bytes)
    if not p_ptr or not o_ptr:
        return unavailable("reference nvshmem_malloc failed")
    partial = torch.as_tensor(_Sym(p_ptr, partial_bytes), device=dev).view(torch.bfloat16).view(M, N)
    out = torch.as_tensor(_Sym(o_ptr, out_bytes), device=dev).view(torch.bfloat16).view(rows, N)

    def step(x, w):
        torch.matmul(x, w.t(), out=partial)
        rc = lib.nvshmemx_bfloat16_sum_reducescatter_on_stream(0, o_ptr, p_ptr, rows * N, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"reference reducescatter returned {rc}")
        return out

    class Stack:
        """L tensor-parallel MLP blocks on the reference's collectives: the token shard lives in a symmetric buffer,
        fcollect gathers it, cuBLAS multiplies, torch applies the GELU, cuBLAS multiplies again into the symmetric
        partial buffer and the reference's reduce-scatter writes the next block's token shard."""

        def __init__(self, layers):
            from bench import HIDDEN
            self.layers = layers
            self.kernels_per_forward = 0  # none of this repository's kernels
            gen = torch.Generator(device=dev)
            gen.manual_seed(99 + rank)
            self.w_up = [torch.empty(K_LOCAL, HIDDEN, device=dev, dtype=torch.float32).normal_(0.0, 0.02, generator=gen).to(torch.bfloat16) for _ in range(layers)]
            self.w_down = [torch.empty(HIDDEN, K_LOCAL, device=dev, dtype=torch.float32).normal_(0.0, 0.02, generator=gen).to(torch.bfloat16) for _ in range(layers)]
            self.s_ptr = lib.nvshmem_malloc(rows * HIDDEN * 2)
            self.g_ptr = lib.nvshmem_malloc(M * HIDDEN * 2)
            self.r_ptrs = [lib.nvshmem_malloc(rows * HIDDEN * 2) for _ in range(2)]
            if not self.s_ptr or not self.g_ptr or not all(self.r_ptrs):
                raise RuntimeError("reference nvshmem_malloc failed")
            self.input_shard = torch.as_tensor(_Sym(self.s_ptr, rows * HIDDEN * 2), device=dev).view(torch.bfloat16).view(rows, HIDDEN)
            self.gathered = torch.as_tensor(_Sym(self.g_ptr, M * HIDDEN * 2), device=dev).view(torch.bfloat16).view(M, HIDDEN)
            self.results = [torch.as_tensor(_Sym(q, rows * HIDDEN * 2), device=dev).view(torch.bfloat16).view(rows, HIDDEN) for q in self.r_ptrs]
            self.h = torch.empty(M, K_LOCAL, device=dev, dtype=torch.bfloat16)
            self.hidden = HIDDEN

        def forward(self, b):
            stream = torch.cuda.current_stream().cuda_stream
            for l in range(self.layers):
                rc = lib.nvshmemx_bfloat16_fcollect_on_stream(0, self.g_ptr, self.s_ptr, rows * self.hidden, stream)
                torch.matmul(self.gathered, self.w_up[l].t(), out=self.h)
                h = torch.nn.functional.gelu(self.h, approximate="tanh")
                torch.matmul(h, self.w_down[l].t(), out=partial)
                dst = self.s_ptr if l + 1 < self.layers else self.r_ptrs[b]
                rc |= lib.nvshmemx_bfloat16_sum_reducescatter_on_stream(0, dst, p_ptr, rows * self.hidden, stream)
                if rc != 0:
                    raise RuntimeError(f"a reference collective returned {rc}")
            return self.results[b]

        def free(self):
            for q in [self.s_ptr, self.g_ptr] + self.r_ptrs:
                lib.nvshmem_free(q)

    stack = Stack(args.layers)
    line = timed_runs(step, stack, args, M, N, K_LOCAL, rank, world, local_rank, launches_per_step=0)
    line["impl"] = "reference"
    line["path"] = ("torch.matmul (cuBLAS) + libnvshmem_host.so nvshmemx_bfloat16_sum_reducescatter_on_stream; end to end: + "
                    "nvshmemx_bfloat16_fcollect_on_stream and torch GELU")
    torch.cuda.synchronize()
    stack.free()
    lib.nvshmem_free(p_ptr)
    lib.nvshmem_free(o_ptr)
    lib.nvshmemx_hostlib_finalize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line
