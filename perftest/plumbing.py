"""Host-only plumbing with no GPU: unique-id bootstrap, heap bring-up on the host-memory back end, a seeded
sequence of 64 malloc / align / free calls (sizes log-uniform in 8 B - 16 MB, alignments 64 / 256 / 4096) whose
offsets must agree on every PE, team creation and barriers.  Prints one JSON line with the wall-clock times.

  python -m nvshmem_b200.launch -n 2 -- python -m perftest.plumbing

(the reference cannot initialise without a GPU, so there is no counterpart to compare with)
"""
from __future__ import annotations

import ctypes as C
import json
import os
import random
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> int:
    os.environ.setdefault("NVSHMEM_HEAP_BACKEND", "HOST")
    from nvshmem_b200.bindings import host as H
    lib = H.load()
    t0 = time.perf_counter()
    lib.nvshmem_init()
    t_init = time.perf_counter() - t0
    me, n = lib.nvshmem_my_pe(), lib.nvshmem_n_pes()
    rng = random.Random(20240611)
    base = lib.nvshmemx_b200_heap_info(0)
    live, trace = [], []
    t0 = time.perf_counter()
    for _ in range(64):
        if live and rng.random() < 0.4:
            p = live.pop(rng.randrange(len(live)))
            lib.nvshmem_free(C.c_void_p(p))
            trace.append(-1)
        else:
            size, align = int(2 ** rng.uniform(3, 24)), rng.choice([64, 256, 4096])
            p = lib.nvshmem_align(align, size)
            if not p:
                print(f"PE {me}: allocation of {size} bytes failed", file=sys.stderr)
                return 1
            live.append(p)
            trace.append(p - base)
    t_alloc = time.perf_counter() - t0
    # every PE's offsets, compared through the heap itself: PE 0 collects them with gets
    words = len(trace)
    table = lib.nvshmem_malloc(8 * words)
    arr = (C.c_long * words)(*trace)
    lib.nvshmem_putmem(C.c_void_p(table), arr, 8 * words, me)
    lib.nvshmem_barrier_all()
    same = True
    if me == 0:
        other = (C.c_long * words)()
        for pe in range(1, n):
            lib.nvshmem_getmem(other, C.c_void_p(table), 8 * words, pe)
            same = same and list(other) == trace
    t0 = time.perf_counter()
    for _ in range(100):
        lib.nvshmem_barrier_all()
    t_barrier = (time.perf_counter() - t0) / 100
    t0 = time.perf_counter()
    team = C.c_int(-1)
    st = lib.nvshmem_team_split_strided(0, 0, 1, n, None, 0, C.byref(team))
    t_team = time.perf_counter() - t0
    if st == 0:
        lib.nvshmem_team_destroy(team.value)
    for p in live:
        lib.nvshmem_free(C.c_void_p(p))
    lib.nvshmem_free(C.c_void_p(table))
    lib.nvshmem_finalize()
    if me == 0:
        print(json.dumps({"test": "host_plumbing", "npes": n, "offsets_identical": same, "init_ms": round(t_init * 1e3, 2), "alloc_sequence_64_ops_ms": round(t_alloc * 1e3, 2),
                          "barrier_us": round(t_barrier * 1e6, 1), "team_split_ms": round(t_team * 1e3, 2), "team_status": st}), flush=True)
    return 0 if same and st == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
