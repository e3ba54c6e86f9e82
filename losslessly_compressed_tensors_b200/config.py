"""Module-level settings, kept for import compatibility with ``LCT/config.py:18-31``.

This build targets one GPU generation (sm_100a) with one set of hand-written
kernels, so the reference's backend/tuning switches have no effect here.  Both
lane mappings of the reference are implemented: ``"swizzle"`` (default, lane
``l`` of row ``n`` holds element ``n*256 + (l ^ (n & 254))``) and ``"linear"``.
As in the reference the mapping is process-wide and must stay fixed while
compressed tensors are in use; unlike the reference it may be assigned at any
time before the codec is used (it is handed to the library on the next launch).
"""
from typing import Literal

lane_mapping: Literal["swizzle", "linear"] = "swizzle"
kernel_backend: str = ""
reset_cache: bool = False
use_tilelang: bool = False
tilelang_verbose: bool = False


def check() -> None:
    """Raise if a setting asks for something this build does not provide."""
    if lane_mapping not in ("swizzle", "linear"):
        raise ValueError("config.lane_mapping must be 'swizzle' or 'linear'")
    if use_tilelang:
        raise ValueError("config.use_tilelang is not supported: there is one CUDA backend")
