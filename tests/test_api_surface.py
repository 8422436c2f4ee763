"""Source compatibility: every function name that the reference's public headers declare (nvshmem.h + nvshmemx.h,
macros expanded) is also declared by this library's headers.  Needs the reference's installed headers under
baseline/_ref/include and nvcc; skipped where either is missing."""
import os
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


def test_flat_bindings_export_the_reference_names():
    """Every public name of the reference's pointer-level Python bindings (nvshmem4py/nvshmem/bindings/nvshmem.pyx:
    `cpdef` functions, classes and enums) is reachable as ``nvshmem.bindings.<name>``.  The list is read from that
    file's text when the reference tree is present, else the test checks the families by pattern."""
    import re
    import nvshmem.bindings as b
    pyx = Path(os.environ.get("BSHMEM_REFERENCE_TREE", str(ROOT.parent / "reference"))) / "nvshmem4py" / "nvshmem" / "bindings" / "nvshmem.pyx"
    if pyx.exists():
        names = set(re.findall(r"^(?:cpdef|def)\s+(?:inline\s+)?(?:[\w\[\]]+\s+)??(\w+)\(", pyx.read_text(), flags=re.M))
        names |= set(re.findall(r"^(?:cdef\s+)?class\s+(\w+)", pyx.read_text(), flags=re.M))
        names = {n for n in names if not n.startswith("_")}
        assert len(names) > 200, len(names)
    else:
        names = {f"{t}_{k}_on_stream" for t in ("float", "half", "bfloat16", "int32", "uint64", "size", "schar") for k in
                 ("alltoall", "broadcast", "fcollect", "sum_reduce", "max_reduce", "min_reducescatter")} | {"malloc", "free", "ptr", "mc_ptr", "Team_id", "InitAttr"}
    missing = sorted(n for n in names if not hasattr(b, n))
    assert not missing, missing


def test_reference_import_paths_name_the_same_modules():
    """``nvshmem.<path>`` and ``nvshmem_b200.<path>`` are one module object each (one copy of the tracking state), and
    the submodule paths of the reference package exist."""
    import importlib
    for path in ("core", "core.memory", "core.collective", "core.rma", "core.teams", "core.direct", "core.init_fini", "core.nvshmem_types", "core.interop.torch",
                 "core.interop.cupy", "bindings", "bindings.nvshmem"):
        assert importlib.import_module("nvshmem." + path) is importlib.import_module("nvshmem_b200." + path), path
    from nvshmem.core.interop.torch import tensor, get_peer_tensor  # noqa: F401
    from nvshmem.bindings import malloc, Team_id  # noqa: F401


def test_every_environment_variable_of_the_reference_is_known():
    """Each NVSHMEM_<NAME> that the reference's option table defines is a row of this library's table (with an effect,
    or listed as accepted without one), so `nvshmem-info -a` documents what a job script's settings do here."""
    ref_defs = Path(os.environ.get("BSHMEM_REFERENCE_TREE", str(ROOT.parent / "reference"))) / "src" / "include"
    if not ref_defs.exists():
        pytest.skip("the reference tree is not present")
    ref = set()
    for p in ref_defs.rglob("*.h"):
        ref |= set(re.findall(r"NVSHMEMI_ENV_DEF\(([A-Z0-9_]+)", p.read_text(errors="replace")))
    ref -= {"NAME"}  # the macro's own parameter name in its definition
    assert len(ref) > 40, len(ref)
    mine = set(re.findall(r"^  X\(([A-Z0-9_]+)", (ROOT / "csrc" / "src" / "util" / "env.h").read_text(), flags=re.M))
    # out-of-scope transports have their own variables in the reference (IB / UCX / libfabric tables are separate files)
    missing = sorted(ref - mine)
    assert not missing, missing
