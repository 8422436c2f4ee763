"""In-tree build of the native libraries with nvcc, for sm_100a only.

Targets (all land in ``nvshmem_b200/lib``):

* ``libbshmem_host.so``   – host library: bootstrap, heap, teams, host API, on-stream collectives
* ``libbshmem_fused.so``  – fused tcgen05 GEMM + collective kernels and the MoE dispatch/combine kernels
* ``libbshmem_devtest.so``– kernels that exercise the device API (used by the test-suite and perftest)
* ``libbshmem_bootstrap_file.so`` / ``_mpi.so`` / ``_shmem.so`` – bootstrap plugins (file exchange; MPI and OpenSHMEM, opened at run time)
* ``nvshmem-info``        – prints version, build options and environment variables

Objects are rebuilt when a source or any header is newer.  ``python -m
nvshmem_b200.utils.build`` builds everything; ``--verbose`` adds ``-Xptxas -v``.

``--sanitize=address|undefined|thread`` (or a comma list such as ``address,undefined``) builds an
instrumented copy of the HOST library and the bootstrap plugin into ``nvshmem_b200/lib-<name>``
(objects under ``build/obj-<name>``); the Python layer loads that copy when ``BSHMEM_LIB_DIR`` names
the directory, and the interpreter needs the sanitizer runtime preloaded (``sanitizer_env`` returns
the environment for a child process).  The CPU test-suite runs a part of itself that way.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
LIB = ROOT / "nvshmem_b200" / "lib"
OBJ = ROOT / "build" / "obj"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function",
          "-I", str(CSRC / "include"), "-I", str(CSRC / "src")]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _headers_mtime() -> float:
    newest = 0.0
    for pat in ("**/*.h", "**/*.cuh", "**/*.hpp"):
        for p in CSRC.glob(pat):
            newest = max(newest, p.stat().st_mtime)
    return newest


def sanitizer_dirs(sanitize: str) -> tuple[Path, Path]:
    tag = sanitize.replace(",", "-")
    return ROOT / "nvshmem_b200" / f"lib-{tag}", ROOT / "build" / f"obj-{tag}"


def sanitizer_env(sanitize: str, log_dir: str | None = None) -> dict[str, str]:
    """Environment for a Python child process that loads the instrumented host library.

    ThreadSanitizer also watches the interpreter, torch and gloo, which are not instrumented, and reports their
    internal locking as errors; those processes therefore exit normally (exitcode=0) and write their reports to
    `log_dir`, where the caller looks for reports that name this library (`tsan_reports_about_us`)."""
    import subprocess as sp
    libs = []
    for s in sanitize.split(","):
        name = {"address": "libasan.so", "undefined": "libubsan.so", "thread": "libtsan.so"}[s]
        libs.append(sp.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip())
    # Instrumented processes run several times slower: the bound of the library's waits grows with them, so that a busy
    # machine shows up as a slow run and not as a peer that "did not arrive".
    env = {"LD_PRELOAD": ":".join(libs), "BSHMEM_LIB_DIR": str(sanitizer_dirs(sanitize)[0]), "NVSHMEM_WAIT_TIMEOUT_MS": "30000",
           "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=1:protect_shadow_gap=0", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1",
           "TSAN_OPTIONS": f"halt_on_error=0:exitcode=0:report_signal_unsafe=0:suppressions={ROOT / 'tests' / 'data' / 'tsan.supp'}"
                           + (f":log_path={log_dir}/tsan" if log_dir else "")}
    return env


def tsan_reports_about_us(log_dir: str) -> list[str]:
    """The ThreadSanitizer reports under `log_dir` that have a frame of this repository's host library."""
    found = []
    for p in sorted(Path(log_dir).glob("tsan.*")):
        text = p.read_text(errors="replace")
        for report in text.split("=================="):
            if "WARNING: ThreadSanitizer" in report and "libbshmem" in report:
                found.append(report.strip())
    return found


def _compile(src: Path, extra: list[str], verbose: bool, hdr_mtime: float, obj_dir: Path | None = None) -> Path:
    rel = src.relative_to(CSRC) if CSRC in src.parents else src.relative_to(ROOT)
    obj = (obj_dir or OBJ) / (str(rel).replace("/", "__") + ".o")
    obj.parent.mkdir(parents=True, exist_ok=True)
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj
    cmd = [nvcc(), "-c", str(src), "-o", str(obj)] + COMMON + extra
    if src.suffix == ".cu":
        cmd += ARCH_FLAGS
        if verbose:
            cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {rel}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr:
        sys.stderr.write(f"--- {rel}\n{res.stderr}\n")
    elif res.stderr.strip():
        # keep warnings visible but short
        lines = [l for l in res.stderr.splitlines() if "warning" in l.lower()]
        if lines:
            sys.stderr.write(f"--- {rel}: {len(lines)} warning(s)\n")
    return obj


def _link(objs: list[Path], out: Path, shared: bool, libs: list[str]) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    if out.exists() and all(out.stat().st_mtime > o.stat().st_mtime for o in objs):
        return
    cmd = [nvcc(), "-o", str(out)] + [str(o) for o in objs] + ARCH_FLAGS + libs
    if shared:
        cmd += ["-shared"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link of {out.name} failed:\n{res.stdout}\n{res.stderr}")


def _sources(*dirs: str) -> list[Path]:
    out: list[Path] = []
    for d in dirs:
        out += sorted((CSRC / "src" / d).glob("*.cpp")) + sorted((CSRC / "src" / d).glob("*.cu"))
    return out


def build_sanitized(sanitize: str, jobs: int | None = None) -> dict[str, Path]:
    """Builds the host library and the bootstrap plugin with -fsanitize=<sanitize> into their own directories."""
    hdr = _headers_mtime()
    jobs = jobs or min(8, os.cpu_count() or 4)
    lib_dir, obj_dir = sanitizer_dirs(sanitize)
    san = [f for s in sanitize.split(",") for f in ("-Xcompiler", f"-fsanitize={s}")]  # nvcc splits -Xcompiler values at commas
    flags = san + ["-Xcompiler", "-fno-omit-frame-pointer", "-g"]
    built = {}
    for name, srcs, out, libs in (
            ("host", _sources("util", "bootstrap", "heap", "team", "state", "transport", "host", "coll"), lib_dir / "libbshmem_host.so",
             ["-ldl", "-lpthread", "-lrt", "-Xlinker", f"--version-script={CSRC / 'bshmem_host.sym'}"]),
            ("plugins", [CSRC / "src" / "bootstrap_plugins" / "bootstrap_file.cpp"], lib_dir / "libbshmem_bootstrap_file.so", []),
            ("plugin_mpi", [CSRC / "src" / "bootstrap_plugins" / "bootstrap_mpi.cpp"], lib_dir / "libbshmem_bootstrap_mpi.so", ["-ldl"]),
            ("plugin_shmem", [CSRC / "src" / "bootstrap_plugins" / "bootstrap_shmem.cpp"], lib_dir / "libbshmem_bootstrap_shmem.so", ["-ldl"])):
        with ThreadPoolExecutor(jobs) as ex:
            objs = list(ex.map(lambda s: _compile(s, flags, False, hdr, obj_dir), srcs))
        _link(objs, out, True, libs + san)
        built[name] = out
    return built


def build_all(verbose: bool = False, jobs: int | None = None, only: str | None = None) -> dict[str, Path]:
    """Builds every native target and returns their paths."""
    hdr = _headers_mtime()
    jobs = jobs or min(8, os.cpu_count() or 4)
    groups = {
        "host": (_sources("util", "bootstrap", "heap", "team", "state", "transport", "host", "coll"), LIB / "libbshmem_host.so", True,
                 ["-ldl", "-lpthread", "-lrt", "-Xlinker", f"--version-script={CSRC / 'bshmem_host.sym'}"]),
        "fused": (_sources("fused"), LIB / "libbshmem_fused.so", True, ["-ldl"]),
        "devtest": (_sources("devtest"), LIB / "libbshmem_devtest.so", True, ["-L", str(LIB), "-lbshmem_host", "-Xlinker", "-rpath=$ORIGIN"]),
        "plugins": ([CSRC / "src" / "bootstrap_plugins" / "bootstrap_file.cpp"], LIB / "libbshmem_bootstrap_file.so", True, []),
        "plugin_mpi": ([CSRC / "src" / "bootstrap_plugins" / "bootstrap_mpi.cpp"], LIB / "libbshmem_bootstrap_mpi.so", True, ["-ldl"]),
        "plugin_shmem": ([CSRC / "src" / "bootstrap_plugins" / "bootstrap_shmem.cpp"], LIB / "libbshmem_bootstrap_shmem.so", True, ["-ldl"]),
        "info": (_sources("tools"), LIB / "nvshmem-info", False, ["-L", str(LIB), "-lbshmem_host", "-Xlinker", "-rpath=$ORIGIN"]),
    }
    built: dict[str, Path] = {}
    if only in (None, "examples") and (ROOT / "examples").is_dir():
        # One program per source file, linked against the host library (run them with `python -m nvshmem_b200.launch`).
        ex_libs = ["-L", str(LIB), "-lbshmem_host", "-lcuda", "-Xlinker", "-rpath=$ORIGIN/../../nvshmem_b200/lib"]
        for src in sorted((ROOT / "examples").glob("*.cu")) + sorted((ROOT / "examples").glob("*.cpp")):
            groups["example:" + src.stem] = ([src], ROOT / "examples" / "bin" / src.stem, False, ex_libs)
    def wanted(name: str) -> bool:
        return not only or name == only or (only == "examples" and name.startswith("example:"))

    def build_group(item):
        name, (srcs, out, shared, libs) = item
        with ThreadPoolExecutor(jobs) as ex:
            objs = list(ex.map(lambda s: _compile(s, [], verbose, hdr), srcs))
        _link(objs, out, shared, libs)
        return name, out

    # The libraries in order (later ones link against the host library), then the one-file example programs side by side.
    for item in groups.items():
        if wanted(item[0]) and item[1][0] and not item[0].startswith("example:"):
            name, out = build_group(item)
            built[name] = out
    examples = [item for item in groups.items() if item[0].startswith("example:") and wanted(item[0])]
    if examples:
        with ThreadPoolExecutor(jobs) as ex:
            for name, out in ex.map(build_group, examples):
                built[name] = out
    return built


def main() -> None:
    verbose = "--verbose" in sys.argv
    only = None
    for a in sys.argv[1:]:
        if a.startswith("--only="):
            only = a.split("=", 1)[1]
        if a.startswith("--sanitize="):
            for name, path in build_sanitized(a.split("=", 1)[1]).items():
                print(f"{name} ({a[2:]}): {path}")
            return
    for name, path in build_all(verbose=verbose, only=only).items():
        print(f"{name}: {path}")


if __name__ == "__main__":
    main()
