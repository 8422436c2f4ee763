"""Import-name compatibility with the reference's Python package: ``import nvshmem.core`` resolves to this
library's Python layer (reference: nvshmem4py/nvshmem/__init__.py)."""
from nvshmem_b200 import core  # noqa: F401
from nvshmem_b200 import bindings  # noqa: F401
import sys as _sys

_sys.modules[__name__ + ".core"] = core
_sys.modules[__name__ + ".bindings"] = bindings
__version__ = "0.1.0"
