"""Module-level settings, kept for import compatibility with ``LCT/config.py:18-31``.

This build targets one GPU generation (sm_100a) with one set of hand-written
kernels, so the reference's backend/tuning switches have no effect here; only
the default lane mapping is implemented and any other value is rejected when
the codec is first used.
"""
from typing import Literal

lane_mapping: Literal["swizzle"] = "swizzle"
kernel_backend: str = ""
reset_cache: bool = False
use_tilelang: bool = False
tilelang_verbose: bool = False


def check() -> None:
    """Raise if a setting asks for something this build does not provide."""
    if lane_mapping != "swizzle":
        raise ValueError("only config.lane_mapping = 'swizzle' is supported")
    if use_tilelang:
        raise ValueError("config.use_tilelang is not supported: there is one CUDA backend")
