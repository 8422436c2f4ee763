"""The programs under examples/ are built by the in-tree build and run through the single-node launcher.
They validate themselves and exit non-zero on a wrong result (the reference uses its examples the same
way: examples/ring-reduce.cu, ring-bcast.cu)."""
import os
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
BIN = ROOT / "examples" / "bin"


def _run(name, n, args=(), env=None, timeout=120):
    from nvshmem_b200.launch import launch
    exe = BIN / name
    assert exe.exists(), f"{exe} is missing: python -m nvshmem_b200.utils.build --only=examples"
    extra = {"NVSHMEM_WAIT_TIMEOUT_MS": "5000", "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000"}
    extra.update(env or {})
    status, outs = launch(n, [str(exe), *args], timeout=timeout, env_extra=extra, capture=True)
    assert status == 0, f"{name} exited {status}:\n" + "\n".join(outs)
    return outs


def test_hello_runs_without_a_gpu_on_the_host_heap():
    outs = _run("hello", 3, env={"NVSHMEM_HEAP_BACKEND": "HOST"})
    text = "".join(outs)
    for pe in range(3):
        assert f"Hello from PE {pe} of 3" in text


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["dev-guide-ring", "collective-launch", "thread-group", "on-stream", "put-block", "ring-bcast", "ring-reduce", "user-buffer"])
def test_example_validates_itself(name):
    n = min(_gpus(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    outs = _run(name, n)
    assert "WRONG" not in "".join(outs)


@pytest.mark.gpu
def test_uid_based_init(tmp_path):
    n = min(_gpus(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    _run("uid-based-init", n, env={"UID_FILE": str(tmp_path / "uid.bin")})
