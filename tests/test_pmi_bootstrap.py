"""PMI-1 and PMI-2 bootstraps against the process manager in baseline/pmi_launcher.py, on CPU (host-memory heap)."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_pmi_bootstrap_collectives_and_full_init():
    from baseline.pmi_launcher import launch
    status, out = launch(3, [sys.executable, str(ROOT / "tests" / "pmi_child.py")], timeout=120,
                         env_extra={"NVSHMEM_BOOTSTRAP": "PMI", "NVSHMEM_HEAP_BACKEND": "HOST", "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000"}, quiet=True)
    assert status == 0, out
    assert "pmi collectives ok on 3 ranks" in out and "full init over pmi ok" in out


def test_pmi2_bootstrap_collectives_and_full_init():
    """The same child under NVSHMEM_BOOTSTRAP_PMI=PMI-2: version negotiation, fullinit, key-value puts, fences, gets."""
    from baseline.pmi_launcher import launch
    status, out = launch(3, [sys.executable, str(ROOT / "tests" / "pmi_child.py")], timeout=120,
                         env_extra={"NVSHMEM_BOOTSTRAP": "PMI", "NVSHMEM_BOOTSTRAP_PMI": "PMI-2", "NVSHMEM_HEAP_BACKEND": "HOST", "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000",
                                    "NVSHMEM_DEBUG": "INFO", "NVSHMEM_DEBUG_SUBSYS": "BOOTSTRAP"}, quiet=True)
    assert status == 0, out
    assert "pmi collectives ok on 3 ranks" in out and "full init over pmi ok" in out
