"""cacti_b200: sm_100a kernels behind a C ABI that replace cacti's Futhark/cuBLAS thunks.

`cacti_b200.capi` is the raw ctypes binding; `cacti_b200.ops` wraps it for torch tensors (torch is
used only as the owner of device memory and streams).
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
