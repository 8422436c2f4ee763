"""Multi-PE GPU tests of the parts that were written last: the MoE dispatch that sends a token once per destination
PE, the recursive-exchange all-reduce, one kernel that calls every queue-pair / sized / byte-collective wrapper
together with the copy-engine collectives on several PEs, and two Python examples.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest

from tests._mp import run_workers
from tests.conftest import gpu_count

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

NG = min(gpu_count(), 8)
need2 = pytest.mark.skipif(gpu_count() < 2, reason="needs two or more GPUs")
NO_NVLS = {"NVSHMEM_DISABLE_NVLS": "1", "NCCL_NVLS_ENABLE": "0"}


@need2
def test_allreduce_by_recursive_exchange():
    run_workers("allreduce_recursive_exchange", NG, gpu=True, env=NO_NVLS, timeout=300)


@need2
def test_device_api_wrappers_and_copy_engine_collectives():
    run_workers("device_api_wrappers_and_copy_engine_collectives", NG, gpu=True, env=NO_NVLS, timeout=300)


@need2
def test_moe_dispatch_once_per_pe():
    run_workers("moe_dispatch_once_per_pe", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
@pytest.mark.parametrize("script", ["on_stream.py", "init_fini.py", "triton_device_api.py"])
def test_late_python_examples_run_on_gpus(script):
    """examples/python/on_stream.py, init_fini.py (which starts and stops the library four times in one process) and
    triton_device_api.py (Triton kernels that signal and wait by themselves) as torchrun jobs on two GPUs; they check
    their own results.  The first two also run on the host heap in the CPU suite; the third compiles there."""
    import os
    import subprocess
    import sys
    from tests._mp import ROOT, free_port
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NVSHMEM_DISABLE_NVLS="1", NVSHMEM_WAIT_TIMEOUT_MS="5000", PYTHONPATH=ROOT)  # no multicast: plain peer stores only
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "examples", "python", script)]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "WRONG" not in res.stdout
