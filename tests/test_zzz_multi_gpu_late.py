"""Multi-PE GPU tests of the parts that were written last: the MoE dispatch that sends a token once per destination
PE, the recursive-exchange all-reduce, and one kernel that calls every queue-pair / sized / byte-collective wrapper
together with the copy-engine collectives on several PEs.

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
