"""Packaging: ``pip install .`` builds the native libraries for sm_100a with nvcc (no GPU needed) and installs the
Python layer with them (``nvshmem_b200`` and the import-name alias ``nvshmem``), the public headers under
``nvshmem_b200/include`` for C++ / CUDA users, and ``nvshmem-info``.  (Role of the reference's nvshmem4py/setup.py
and of its CMake install rules.)"""
import shutil
from pathlib import Path

from setuptools import Distribution, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


class BuildWithNative(build_py):
    """Runs the in-tree native build first and copies the public headers into the package."""

    def run(self):
        import sys
        sys.path.insert(0, str(ROOT))
        from nvshmem_b200.utils.build import build_all
        for name in ("host", "fused", "devtest", "plugins", "plugin_mpi", "plugin_shmem", "info"):
            build_all(only=name)
        dst = ROOT / "nvshmem_b200" / "include"
        if dst.exists():
            shutil.rmtree(dst)
        shutil.copytree(ROOT / "csrc" / "include", dst)
        super().run()


class BinaryDistribution(Distribution):
    """The wheel carries shared libraries built for this platform."""

    def has_ext_modules(self):
        return True


setup(
    distclass=BinaryDistribution,
    name="nvshmem-b200",
    version="0.2.0",
    description="B200-native PGAS communication library with NVSHMEM's API: symmetric heap over CUDA VMM, device-initiated RMA, NVLS collectives, fused tcgen05 GEMM + collective kernels",
    packages=find_packages(include=["nvshmem_b200", "nvshmem_b200.*", "nvshmem", "perftest"]),
    package_data={"nvshmem_b200": ["lib/*.so", "lib/nvshmem-info", "include/*.h", "include/bshmem/*"]},
    python_requires=">=3.10",
    install_requires=["numpy"],
    extras_require={"torch": ["torch"]},
    cmdclass={"build_py": BuildWithNative},
    entry_points={"console_scripts": ["nvshmem-b200-launch=nvshmem_b200.launch:main"]},
    zip_safe=False,
)
