"""Import-name compatibility with the reference's Python package: ``import nvshmem.core``, ``nvshmem.bindings`` and
every submodule path below them resolve to the SAME module objects as ``nvshmem_b200.core`` / ``nvshmem_b200.bindings``
(reference: nvshmem4py/nvshmem/__init__.py).  A finder maps the names instead of importing the files a second time,
so there is one copy of the library state whichever name a program uses."""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys as _sys

_REAL = "nvshmem_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        real = _REAL + fullname[len(__name__):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.machinery.ModuleSpec(fullname, self)

    def create_module(self, spec):
        return importlib.import_module(_REAL + spec.name[len(__name__):])

    def exec_module(self, module):
        pass


_sys.meta_path.insert(0, _AliasFinder())
from nvshmem_b200 import core, bindings  # noqa: E402,F401

_sys.modules[__name__ + ".core"] = core
_sys.modules[__name__ + ".bindings"] = bindings
__version__ = "0.1.0"
