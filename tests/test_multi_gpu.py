"""Multi-PE tests on real GPUs: one child process per GPU (as many as the box has, up to 8), NCCL only for the
test harness' own gathers.  NVLS is off unless a test is about it; the tests about it leave through the
harness' soft exit (a failing rank detaches from the multicast objects before it goes)."""
import pytest

from tests._mp import run_workers
from tests.conftest import gpu_count

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

NG = min(gpu_count(), 8)
need4 = pytest.mark.skipif(gpu_count() < 4, reason="needs four or more GPUs")
NVLS_ON = {"NCCL_NVLS_ENABLE": "0"}  # this library's multicast windows on, NCCL's own NVLS off
need2 = pytest.mark.skipif(gpu_count() < 2, reason="needs two or more GPUs")
NO_NVLS = {"NVSHMEM_DISABLE_NVLS": "1", "NCCL_NVLS_ENABLE": "0"}


@need2
def test_alloc_symmetry_gpu():
    run_workers("alloc_symmetry", NG, gpu=True, env=NO_NVLS)


@need2
def test_host_rma_and_atomics_gpu():
    run_workers("host_rma_and_atomics", NG, gpu=True, env=NO_NVLS)


@need2
def test_teams_gpu():
    run_workers("teams", NG, gpu=True, env=NO_NVLS)


@need2
def test_device_rma():
    run_workers("device_rma", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
def test_device_signals_atomics_barriers():
    run_workers("device_signals_amo_barrier", NG, gpu=True, env=NO_NVLS, timeout=240)


@need2
def test_collectives_on_stream():
    run_workers("collectives_on_stream", NG, gpu=True, env=NO_NVLS, timeout=900)


@need2
def test_collectives_on_stream_nvls():
    run_workers("collectives_on_stream", NG, gpu=True, env={"NCCL_NVLS_ENABLE": "0"}, timeout=900)


@need2
def test_collectives_in_cuda_graph():
    run_workers("collectives_in_graph", NG, gpu=True, env=NO_NVLS)


@need2
def test_device_collectives_and_tiles():
    run_workers("device_collectives_and_tiles", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
def test_fused_gemm_collectives():
    run_workers("fused_gemm_collectives", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
def test_fused_gemm_collectives_nvls():
    """Switch path: partial tiles reduced with multimem.ld_reduce, the all-reduce's multimem.st epilogue."""
    run_workers("fused_gemm_collectives", NG, gpu=True, env=dict(NVLS_ON, BSHMEM_EXPECT_SWITCH_PATH="1"), timeout=600)


@need2
def test_tp_mlp_stack_nvls():
    run_workers("tp_mlp_stack_matches_fp32_reference", NG, gpu=True, env=NVLS_ON, timeout=600)


@need2
def test_tp_mlp_stack_push_path():
    run_workers("tp_mlp_stack_matches_fp32_reference", NG, gpu=True, env=NO_NVLS, timeout=600)


@need4
def test_team_multicast_windows():
    run_workers("team_multicast_windows", NG - NG % 2, gpu=True, env=NVLS_ON, timeout=600)


@need2
def test_device_collectives_and_tiles_nvls():
    run_workers("device_collectives_and_tiles", NG, gpu=True, env=NVLS_ON, timeout=600)


@need2
def test_moe_dispatch_combine_nvls():
    run_workers("moe_dispatch_combine", NG, gpu=True, env=NVLS_ON, timeout=600)


@need2
def test_moe_dispatch_combine():
    run_workers("moe_dispatch_combine", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
def test_tp_mlp_matches_single_device():
    run_workers("tp_mlp_matches_single_device", NG, gpu=True, env=NO_NVLS, timeout=600)


@need2
def test_device_module_via_driver_api():
    run_workers("device_module_via_driver_api", NG, gpu=True, env=NO_NVLS, timeout=300)


@need2
@pytest.mark.parametrize("script", ["torch_interop.py", "triton_interop.py", "tp_and_ep_blocks.py", "external_memory.py"])
def test_python_examples_run_on_gpus(script):
    """The example programs under examples/python, each as a torchrun job on two GPUs; they check their own results."""
    import os
    import subprocess
    import sys
    from tests._mp import ROOT, free_port
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NVSHMEM_WAIT_TIMEOUT_MS="5000", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "examples", "python", script)]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "WRONG" not in res.stdout


@need2
def test_rank_leaves_between_steps():
    run_workers("rank_leaves_between_steps", NG, gpu=True, env=NO_NVLS)
