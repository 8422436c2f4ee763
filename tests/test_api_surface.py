"""Source compatibility: every function name that the reference's public headers declare (nvshmem.h + nvshmemx.h,
macros expanded) is also declared by this library's headers.  Needs the reference's installed headers under
baseline/_ref/include and nvcc; skipped where either is missing."""
import re
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF_INC = ROOT / "baseline" / "_ref" / "include"
# Names that exist in the reference only through a typo in its size list ("6" where 16 is meant).
KNOWN_REFERENCE_TYPOS = {"nvshmemx_put6_signal_block", "nvshmemx_put6_signal_nbi_block", "nvshmemx_put6_signal_nbi_warp", "nvshmemx_put6_signal_warp"}


def _names(cmd, src):
    out = subprocess.run(cmd + [str(src)], capture_output=True, text=True, timeout=300).stdout
    return set(re.findall(r"\b(nvshmemx?_[A-Za-z0-9_]+)\s*\(", out))


def test_every_reference_function_name_is_declared(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not (REF_INC / "nvshmem.h").exists() or not Path(nvcc).exists() or not shutil.which("g++"):
        pytest.skip("needs baseline/_ref/include, nvcc and g++")
    src = tmp_path / "api.cu"
    src.write_text('#include "nvshmem.h"\n#include "nvshmemx.h"\n')
    cuda_inc = str(Path(nvcc).resolve().parents[1] / "include")
    ref = _names(["g++", "-E", "-x", "c++", "-I", str(REF_INC), "-I", cuda_inc], src)
    mine = _names([nvcc, "-E", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(ROOT / "csrc" / "include")], src)
    assert len(ref) > 2500, "the reference headers did not expand"
    missing = sorted(ref - mine - KNOWN_REFERENCE_TYPOS)
    assert not missing, f"{len(missing)} names of the reference API are not declared: {missing[:20]}"


# The names the reference's Python package exports from ``nvshmem.core`` (union of the ``__all__`` lists of
# nvshmem4py/nvshmem/core/{collective,direct,init_fini,memory,rma,teams,nvshmem_types}.py and interop/{torch,cupy}.py).
NVSHMEM4PY_NAMES = """
BufferTypes ComparisonType InitStatus MutableEnum NvshmemError NvshmemInvalid NvshmemKernelObject NvshmemResource
NvshmemStream NvshmemStreamsType SignalOp TeamConfig TeamUniqueId Teams UniqueID Version
alltoall array array_get_buffer barrier barrier_all broadcast buffer bytearray
bytetensor collective_on_buffer fcollect finalize free free_array free_tensor get
get_multicast_array get_multicast_buffer get_multicast_tensor get_peer_array get_peer_buffer get_peer_tensor get_team_unique_id get_unique_id
get_version init init_status library_finalize library_init module_finalize module_init my_pe
n_pes put put_signal quiet reduce reducescatter register_external_array register_external_buffer
register_external_tensor signal_op signal_wait sync sync_all team_destroy team_init team_my_pe
team_n_pes team_split_2d team_split_strided team_translate_pe tensor tensor_get_buffer unregister_external_array unregister_external_buffer
unregister_external_tensor
""".split()


def test_python_layer_exports_the_reference_names():
    import nvshmem.core as core  # the alias package resolves to nvshmem_b200.core
    import nvshmem_b200.core as mine
    assert core is mine
    missing = [n for n in NVSHMEM4PY_NAMES if not hasattr(core, n)]
    assert not missing, missing
