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
