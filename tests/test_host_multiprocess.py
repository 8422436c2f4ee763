"""Host-side logic as real OS processes on CPU: bootstrap, heap bookkeeping, host RMA, atomics, teams,
and host-made failures.  No GPU is used (gloo backend, host-memory heap)."""
import pytest

from tests._mp import run_workers


@pytest.mark.parametrize("n", [1, 2, 3, 8])
def test_bootstrap_collectives(n):
    run_workers("bootstrap_raw", n)


@pytest.mark.parametrize("n", [2, 4])
def test_alloc_symmetry_seeded_sequence(n):
    run_workers("alloc_symmetry", n, env={"NVSHMEM_SYMMETRIC_SIZE": "8M"})


def test_alloc_symmetry_with_error_checks():
    run_workers("alloc_symmetry", 2, env={"NVSHMEM_SYMMETRIC_SIZE": "8M", "NVSHMEM_ENABLE_ERROR_CHECKS": "1"})


@pytest.mark.parametrize("n", [2, 3])
def test_host_rma_and_atomics(n):
    run_workers("host_rma_and_atomics", n)


@pytest.mark.parametrize("n", [1, 2, 5])
def test_teams(n):
    run_workers("teams", n)


def test_root_drops_a_registration_everyone_times_out():
    run_workers("bootstrap_missing_rank", 3, env={"NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "1500"}, timeout=120)


def test_rank_that_never_joins_gives_error_status():
    run_workers("rank_never_joins", 3, env={"NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "1500"}, timeout=120)


@pytest.mark.parametrize("n", [2, 3])
def test_python_layer_on_host_heap(n):
    run_workers("python_layer_on_host_heap", n)


@pytest.mark.parametrize("n", [2, 3, 4])
def test_collectives_on_host_heap(n):
    run_workers("collectives_on_host_heap", n)


def test_typed_host_api_all_types():
    run_workers("typed_host_api_all_types", 3)


def test_host_atomics_all_types():
    run_workers("host_atomics_all_types", 4)



@pytest.mark.parametrize("n", [1, 3])
def test_flat_bindings_on_host_heap(n):
    run_workers("flat_bindings_on_host_heap", n)


@pytest.mark.parametrize("mode,n", [("none", 4), ("full", 4), ("over", 3)])
def test_several_pes_per_gpu_status(mode, n):
    """LIMITED without an MPS server or with shares above 100 %, FULL with an MPS server and shares that fit; the PE
    that has a GPU to itself (n = 3) reports the ordinary status."""
    run_workers("several_pes_per_gpu_status", n, env={"MPG_MODE": mode})
