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
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    n = 2
    outs = _run(name, n)
    assert "WRONG" not in "".join(outs)


@pytest.mark.gpu
def test_uid_based_init(tmp_path):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    n = 2
    _run("uid-based-init", n, env={"UID_FILE": str(tmp_path / "uid.bin")})


def test_launcher_reports_the_first_failure_and_stops_the_other_ranks():
    import sys
    import time
    from nvshmem_b200.launch import launch
    code = ("import os, sys, time\n"
            "r = int(os.environ['RANK']); assert os.environ['WORLD_SIZE'] == '3' and os.environ['LOCAL_RANK'] == str(r)\n"
            "assert os.environ['NVSHMEM_BOOTSTRAP_UID_SESSION_ID'].startswith('127.0.0.1:')\n"
            "sys.exit(7) if r == 1 else time.sleep(60)\n")
    t0 = time.time()
    status, outs = launch(3, [sys.executable, "-c", code], timeout=50, capture=True)
    assert status == 7 and time.time() - t0 < 30  # the sleeping ranks were terminated, not waited for


def test_launcher_times_out():
    import sys
    from nvshmem_b200.launch import launch
    status, _ = launch(2, [sys.executable, "-c", "import time; time.sleep(60)"], timeout=1.5, capture=True)
    assert status == 124


def test_host_plumbing_benchmark_runs_without_a_gpu():
    """Config (a): bootstrap, host-heap bring-up, the seeded 64-call allocation sequence, barriers, a team."""
    import json
    import sys
    from nvshmem_b200.launch import launch
    status, outs = launch(2, [sys.executable, "-m", "perftest.plumbing"], timeout=120, capture=True,
                          env_extra={"NVSHMEM_HEAP_BACKEND": "HOST", "PYTHONPATH": str(ROOT)})
    assert status == 0, outs
    row = json.loads([l for l in "".join(outs).splitlines() if l.startswith("{")][0])
    assert row["offsets_identical"] is True and row["npes"] == 2 and row["team_status"] == 0


def test_stray_connections_do_not_disturb_the_bootstrap():
    import sys
    from nvshmem_b200.launch import launch
    status, outs = launch(3, [sys.executable, str(ROOT / "tests" / "stray_child.py")], timeout=120, capture=True,
                          env_extra={"NVSHMEM_HEAP_BACKEND": "HOST", "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000"})
    assert status == 0, outs
    assert "bootstrap survived the strays" in "".join(outs)


def test_bootstrap_plugin_is_loaded_and_carries_a_job(tmp_path):
    """NVSHMEM_BOOTSTRAP=PLUGIN with the file-exchange plugin: the whole bring-up (node info, heap, teams, barriers)
    runs over a plugin's allgather / alltoall / barrier."""
    import sys
    from nvshmem_b200.bindings import host as H
    from nvshmem_b200.launch import launch
    plugin = H.lib_path("libbshmem_bootstrap_file.so")
    assert plugin.exists(), "python -m nvshmem_b200.utils.build --only=plugins"
    env = {"NVSHMEM_BOOTSTRAP": "PLUGIN", "NVSHMEM_BOOTSTRAP_PLUGIN": str(plugin), "BSHMEM_FILE_BOOTSTRAP_DIR": str(tmp_path),
           "NVSHMEM_HEAP_BACKEND": "HOST", "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000", "PYTHONPATH": str(ROOT)}
    status, outs = launch(3, [sys.executable, "-m", "perftest.plumbing"], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert '"offsets_identical": true' in "".join(outs)
    leftovers = [p.name for p in tmp_path.iterdir()]
    assert leftovers == [], leftovers  # every rank removed its files


def test_bootstrap_plugin_errors_are_reported(tmp_path):
    import sys
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP": "PLUGIN", "NVSHMEM_BOOTSTRAP_PLUGIN": str(tmp_path / "no_such_plugin.so"), "NVSHMEM_HEAP_BACKEND": "HOST", "PYTHONPATH": str(ROOT)}
    status, outs = launch(1, [sys.executable, "-m", "perftest.plumbing"], timeout=60, capture=True, env_extra=env)
    assert status != 0 and "dlopen" in "".join(outs)


def test_bootstrap_plugin_collectives(tmp_path):
    import sys
    from nvshmem_b200.bindings import host as H
    from nvshmem_b200.launch import launch
    env = {"NVSHMEM_BOOTSTRAP_PLUGIN": str(H.lib_path("libbshmem_bootstrap_file.so")), "BSHMEM_FILE_BOOTSTRAP_DIR": str(tmp_path), "NVSHMEM_BOOTSTRAP_TIMEOUT_MS": "30000"}
    status, outs = launch(4, [sys.executable, str(ROOT / "tests" / "plugin_child.py")], timeout=120, capture=True, env_extra=env)
    assert status == 0, outs
    assert "plugin collectives ok" in "".join(outs) and list(tmp_path.iterdir()) == []


@pytest.mark.parametrize("script", ["init_fini.py", "on_stream.py"])
def test_python_examples_run_on_the_host_heap(script):
    """examples/python/init_fini.py (four ways to start and stop, one after the other in the same processes) and
    on_stream.py as torchrun jobs of three processes with no GPU; they check their own results."""
    import os
    import subprocess
    import sys
    from tests._mp import free_port
    env = dict(os.environ, NVSHMEM_HEAP_BACKEND="HOST", PYTHONPATH=str(ROOT), NVSHMEM_BOOTSTRAP_TIMEOUT_MS="30000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           str(ROOT / "examples" / "python" / script)]
    res = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "WRONG" not in res.stdout and res.stdout.count(" ok") >= 3
