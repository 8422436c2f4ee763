import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices (runs child processes, one per GPU)")


@pytest.fixture(scope="session")
def hostlib():
    from nvshmem_b200.utils.build import build_all
    from nvshmem_b200.bindings import host as H
    if not H.lib_path().exists():
        build_all(only="host")
    return H.load()


def gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0
