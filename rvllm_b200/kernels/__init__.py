"""Access to the kernel library of the product path."""
from __future__ import annotations

from typing import Optional

from ..errors import KernelError
from .library import CudaKernels, AttentionMeta

_library = None


def get_library(device="cuda:0"):
    """The kernel library for `device`.  Only CUDA devices have one; asking for another device
    fails loudly unless a library object was installed with `set_library` (tests do that to
    check host-side logic without a GPU)."""
    global _library
    if _library is not None:
        return _library
    if not str(device).startswith("cuda"):
        raise KernelError(f"no kernels for device {device!r}: the engine runs on CUDA (sm_100a) only")
    _library = CudaKernels(device)
    return _library


def set_library(lib) -> None:
    global _library
    _library = lib
