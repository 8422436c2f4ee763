"""Import paths of the reference package's interop modules (nvshmem4py/nvshmem/core/interop/{torch,cupy}.py): the
functions themselves live in ``core.memory`` (torch) and ``core.compat`` (CuPy)."""
from . import torch, cupy  # noqa: F401
