"""The MPI and OpenSHMEM bootstrap plugins on CPU.  Neither is installed here, so the tests build stand-ins:
tests/data/fake_mpi.c (the entry points the MPI plugin uses, over files), once with each of the two binary
interfaces that the plugin speaks (integer handles of the MPICH family, pointer handles of Open MPI; the stand-in
aborts on a handle that does not belong to its interface, so a mix-up fails the test), and tests/data/fake_shmem.c
(symmetric heaps as shared file mappings)."""
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc to build the stand-in MPI library")


@pytest.fixture(scope="module")
def fake_mpi(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_mpi")
    libs = {}
    for abi, flags in (("mpich", []), ("ompi", ["-DFAKE_OMPI"])):
        so = out / f"libmpi_{abi}.so"
        subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-w", *flags, "-o", str(so), str(ROOT / "tests" / "data" / "fake_mpi.c")], check=True)
        libs[abi] = so
    return libs


def _plugin():
    from nvshmem_b200.bindings import host as H
    p = H.lib_path("libbshmem_bootstrap_mpi.so")
    if not p.exists():
        from nvshmem_b200.utils.build import build_all
        build_all(only="host")
        build_all(only="plugin_mpi")
    return p


@pytest.mark.parametrize("abi", ["mpich", "ompi"])
def test_mpi_plugin_collectives(abi, fake_mpi, tmp_path):
    """allgather / alltoall / barrier with odd and large sizes straight through the plugin's table."""
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP_PLUGIN": str(_plugin()), "NVSHMEM_BOOTSTRAP_MPI_LIB": str(fake_mpi[abi]), "FAKE_MPI_DIR": str(tmp_path)}
    status, outs = launch(4, [sys.executable, str(ROOT / "tests" / "plugin_child.py")], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert "plugin collectives ok" in "".join(outs)
    assert sorted(p.name for p in tmp_path.glob("finalized.*")) == [f"finalized.{r}" for r in range(4)]  # the plugin initialised MPI, so it finalised it


@pytest.mark.parametrize("abi", ["mpich", "ompi"])
def test_mpi_bootstrap_carries_a_job(abi, fake_mpi, tmp_path):
    """NVSHMEM_BOOTSTRAP=MPI: plain nvshmem_init() brings the job up over the MPI library (found by name beside the
    host library, MPI opened from NVSHMEM_BOOTSTRAP_MPI_LIB): node info, heap, teams, barriers."""
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP": "MPI", "NVSHMEM_BOOTSTRAP_MPI_LIB": str(fake_mpi[abi]), "FAKE_MPI_DIR": str(tmp_path), "NVSHMEM_HEAP_BACKEND": "HOST",
           "PYTHONPATH": str(ROOT)}
    status, outs = launch(3, [sys.executable, "-m", "perftest.plumbing"], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert '"offsets_identical": true' in "".join(outs)
    assert len(list(tmp_path.glob("finalized.*"))) == 3


@pytest.mark.parametrize("abi,core_layer", [("mpich", "0"), ("ompi", "0"), ("mpich", "1"), ("ompi", "1")])
def test_init_with_the_programs_communicator(abi, core_layer, fake_mpi, tmp_path):
    """NVSHMEMX_INIT_WITH_MPI_COMM: the program owns MPI, passes the address of its communicator (through the
    pointer-level bindings, or ``nvshmem.core.init(mpi_comm=...)``), and MPI is still alive after the library has shut down."""
    from nvshmem_b200.launch import launch
    env = {"FAKE_MPI_LIB": str(fake_mpi[abi]), "FAKE_MPI_ABI": abi, "FAKE_MPI_DIR": str(tmp_path), "NVSHMEM_HEAP_BACKEND": "HOST", "PYTHONPATH": str(ROOT),
           "USE_CORE_LAYER": core_layer}
    status, outs = launch(3, [sys.executable, str(ROOT / "tests" / "mpi_comm_child.py")], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert "".join(outs).count("init with the program's communicator ok") == 3


def test_mpi_bootstrap_without_an_mpi_library_says_so(tmp_path):
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP": "MPI", "NVSHMEM_BOOTSTRAP_MPI_LIB": str(tmp_path / "no_such_libmpi.so"), "NVSHMEM_HEAP_BACKEND": "HOST", "PYTHONPATH": str(ROOT)}
    status, outs = launch(1, [sys.executable, "-m", "perftest.plumbing"], timeout=60, capture=True, env_extra=env)
    assert status != 0 and "NVSHMEM_BOOTSTRAP_MPI_LIB" in "".join(outs)


# ---------------------------------------------------------------------------------------------- OpenSHMEM
@pytest.fixture(scope="module")
def fake_shmem(tmp_path_factory):
    so = tmp_path_factory.mktemp("fake_shmem") / "liboshmem_fake.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-w", "-o", str(so), str(ROOT / "tests" / "data" / "fake_shmem.c")], check=True)
    return so


def _shmem_plugin():
    from nvshmem_b200.bindings import host as H
    p = H.lib_path("libbshmem_bootstrap_shmem.so")
    if not p.exists():
        from nvshmem_b200.utils.build import build_all
        build_all(only="host")
        build_all(only="plugin_shmem")
    return p


def test_shmem_plugin_collectives(fake_shmem, tmp_path):
    """allgather / alltoall / barrier with odd and large sizes over puts and barriers of the OpenSHMEM library, which
    the plugin opens and therefore initialises and finalises itself."""
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP_PLUGIN": str(_shmem_plugin()), "NVSHMEM_BOOTSTRAP_SHMEM_LIB": str(fake_shmem), "FAKE_SHMEM_DIR": str(tmp_path)}
    status, outs = launch(4, [sys.executable, str(ROOT / "tests" / "plugin_child.py")], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert "plugin collectives ok" in "".join(outs)
    assert len(list(tmp_path.glob("finalized.*"))) == 4


def test_shmem_bootstrap_carries_a_job(fake_shmem, tmp_path):
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP": "SHMEM", "NVSHMEM_BOOTSTRAP_SHMEM_LIB": str(fake_shmem), "FAKE_SHMEM_DIR": str(tmp_path), "NVSHMEM_HEAP_BACKEND": "HOST",
           "PYTHONPATH": str(ROOT)}
    status, outs = launch(3, [sys.executable, "-m", "perftest.plumbing"], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert '"offsets_identical": true' in "".join(outs)


def test_init_beside_the_programs_openshmem(fake_shmem, tmp_path):
    """NVSHMEMX_INIT_WITH_SHMEM: the program has initialised OpenSHMEM; the bootstrap uses it and leaves it running."""
    from nvshmem_b200.launch import launch
    env = {"FAKE_SHMEM_LIB": str(fake_shmem), "FAKE_SHMEM_DIR": str(tmp_path), "NVSHMEM_HEAP_BACKEND": "HOST", "PYTHONPATH": str(ROOT)}
    status, outs = launch(3, [sys.executable, str(ROOT / "tests" / "shmem_child.py")], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert "".join(outs).count("init beside the program's OpenSHMEM ok") == 3
