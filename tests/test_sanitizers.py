"""The host library under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer.

`python -m nvshmem_b200.utils.build --sanitize=<name>` builds an instrumented copy of the host library; the tests
below run the CPU parts of this suite (allocator, option parser, bootstrap sockets, unique-id and PMI bootstraps,
file-descriptor exchange, teams and collectives on the host-memory heap, as child processes over gloo) against it.
Building an instrumented library takes a few minutes, so these runs are opt-in:

    BSHMEM_RUN_SANITIZERS=1 python -m pytest tests/test_sanitizers.py -q

Without the variable only the plumbing (directories, child environment) is checked.
"""
import os
import subprocess
import sys

import pytest

from nvshmem_b200.utils import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WANTED = os.environ.get("BSHMEM_RUN_SANITIZERS") == "1"


def test_sanitizer_builds_live_apart_from_the_ordinary_build():
    lib, obj = build.sanitizer_dirs("address,undefined")
    assert lib.name == "lib-address-undefined" and obj.name == "obj-address-undefined" and lib != build.LIB
    env = build.sanitizer_env("thread", "/tmp/x")
    assert env["LD_PRELOAD"].endswith("libtsan.so") and env["BSHMEM_LIB_DIR"].endswith("lib-thread") and "log_path=/tmp/x/tsan" in env["TSAN_OPTIONS"]


def test_only_reports_with_a_frame_of_this_library_count(tmp_path):
    (tmp_path / "tsan.1").write_text("==================\nWARNING: ThreadSanitizer: data race (pid=1)\n  #0 f (libtorch_cpu.so+0x1)\n==================\n"
                                     "WARNING: ThreadSanitizer: data race (pid=1)\n  #0 g (libbshmem_host.so+0x2)\n==================\n")
    ours = build.tsan_reports_about_us(str(tmp_path))
    assert len(ours) == 1 and "libbshmem_host.so" in ours[0]


def _run_suite_under(sanitize: str, files: list[str], extra: list[str], log_dir=None):
    build.build_sanitized(sanitize)
    env = dict(os.environ, **build.sanitizer_env(sanitize, log_dir))
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider"] + files + extra
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=3000)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]


@pytest.mark.skipif(not WANTED, reason="set BSHMEM_RUN_SANITIZERS=1 (builds an instrumented library first: minutes)")
def test_cpu_suite_under_address_and_undefined_behaviour_sanitizers():
    _run_suite_under("address,undefined", ["tests/test_allocator_properties.py", "tests/test_host_units.py", "tests/test_host_multiprocess.py"],
                     ["--deselect", "tests/test_host_units.py::test_nvshmem_info_tool"])  # the tool is not part of the instrumented build


@pytest.mark.skipif(not WANTED, reason="set BSHMEM_RUN_SANITIZERS=1 (builds an instrumented library first: minutes)")
def test_threaded_parts_under_thread_sanitizer(tmp_path):
    """The parts with threads of their own: the unique-id bootstrap's root thread, the watchdog, the socket layer.
    Reports are collected from every process of the run; only those with a frame of this library count."""
    _run_suite_under("thread", ["tests/test_host_units.py", "tests/test_host_multiprocess.py"], ["--deselect", "tests/test_host_units.py::test_nvshmem_info_tool"], log_dir=str(tmp_path))
    ours = build.tsan_reports_about_us(str(tmp_path))
    assert not ours, "\n\n".join(ours[:3])[:6000]
