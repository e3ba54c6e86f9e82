"""ctypes binding of ``liblct_b200.so`` (declared in ``include/lct_b200.h``).

There is exactly one implementation of every operation: the CUDA library.  If
it has not been built, or cannot be loaded, importing fails with instructions;
nothing falls back to PyTorch or the CPU.
"""
from __future__ import annotations

import ctypes
import os

_PACKAGE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# LCT_B200_LIBRARY points at an alternative build of the same library (e.g. a debug build).
LIBRARY_PATH = os.environ.get("LCT_B200_LIBRARY") or os.path.join(_PACKAGE, "liblct_b200.so")

_p = ctypes.c_void_p
_i = ctypes.c_int
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64


class Overflow(ctypes.Structure):
    """``struct lct_overflow``."""

    _fields_ = [
        ("lanes", _p), ("starts", _p), ("tail", _p), ("descriptor", _p), ("count", _p),
        ("blocks", _p), ("base", _i64), ("mode", _i32), ("reserved", _i32),
    ]


class Operand(ctypes.Structure):
    """``struct lct_operand``."""

    _fields_ = [
        ("encoded", _p), ("side", _p), ("shifted_decode", _p), ("center", _p),
        ("pair_table", _p), ("overflow", Overflow),
    ]


class DecodeJob(ctypes.Structure):
    """``struct lct_decode_job``."""

    _fields_ = [("operand", Operand), ("out", _p), ("size", _i64), ("logical_numel", _i64),
                ("first_block", _i64), ("side_stage", _p)]


class UpdateJob(ctypes.Structure):
    """``struct lct_update_job``."""

    _fields_ = [("a", Operand), ("other", _p), ("known_values", _p), ("result_values", _p),
                ("side_out", _p), ("encoded_out", _p), ("spill", _p), ("center", _p),
                ("shifted_decode", _p), ("counts", _p), ("descriptor", _p), ("blocks_out", _p),
                ("size", _i64), ("logical_numel", _i64), ("first_block", _i64), ("dense_out", _p)]


class EncodeJob(ctypes.Structure):
    """``struct lct_encode_job``."""

    _fields_ = [("src", _p), ("side", _p), ("encoded", _p), ("center", _p), ("shifted_decode", _p),
                ("counts", _p), ("descriptor", _p), ("blocks_out", _p), ("size", _i64),
                ("logical_numel", _i64), ("first_block", _i64)]


_SIGNATURES = {
    "lct_build_pair_table": [_p, _i, _p, _p],
    "lct_center_and_tables": [_p, _i64, _i, _p, _p, _p, _p, _p, _p],
    "lct_shift_tables": [_p, _p, _p, _p, _p, _p],
    "lct_encode": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _i, _i, _p],
    "lct_encode_noalloc": [_p, _p, _p, _p, _p, _i64, _i64, _i, _i, _i, _i, _p],
    "lct_scan_allocate": [_p, _p, _p, _p, _i64, _i, _p],
    "lct_compact_tails": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _i, _p],
    "lct_decode": [ctypes.POINTER(Operand), _p, _i64, _i64, _i, _i, _i, _i, _p],
    "lct_decode_batch": [_p, _i, _i64, _i, _i, _i, _i, _p],
    "lct_set_lane_mapping": [_i],
    "lct_get_lane_mapping": [],
    "lct_compress": [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i64, _i64,
                     _i, _i, _i, _p],
    "lct_compress_batch": [_p, _i, _i64, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _p],
    "lct_pointwise": [ctypes.POINTER(Operand), _p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _i64,
                      _i, _i, _i, _i, _p],
    "lct_update_sample": [ctypes.POINTER(Operand), _p, _p, _p, _i, _i, _i, _p, _p, _p, _i64, _i64,
                          _i, _i, _i, _i, _p],
    "lct_update_fused": [ctypes.POINTER(Operand), _p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _p,
                         _i64, _i64, _i, _i, _i, _i, _p],
    "lct_update": [ctypes.POINTER(Operand), _p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p,
                   _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i64, _i64, _i, _i, _i, _i, _p],
    "lct_update_emit": [ctypes.POINTER(Operand), _p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p,
                        _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i64, _i64, _i, _i, _i, _i, _p,
                        _i, _p, _p, _p],
    "lct_update_batch": [_p, _i, _i64, _p, _p, _i, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i,
                         _i, _i, _p],
    "lct_update_batch_emit": [_p, _i, _i64, _p, _p, _i, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _i,
                              _i, _i, _i, _i, _p],
    "lct_dual_scale_add": [ctypes.POINTER(Operand), ctypes.POINTER(Operand), _p, _p, _p, _i,
                           _i64, _i64, _i, _i, _i, _i, _p],
    "lct_buffer_reset": [_p, _i, _i32, _p],
    "lct_buffer_allocate": [_p, _p, _p, _i, _p, _i, _p],
    "lct_buffer_free": [_p, _p, _p, _i, _p],
    "lct_buffer_free_many": [_p, _p, _i, _p, _i, _p],
}

EXPORTS = tuple(_SIGNATURES) + ("lct_version", "lct_error_string")

_library = None


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise with build instructions if it is absent."""
    global _library
    if _library is not None:
        return _library
    if not os.path.exists(LIBRARY_PATH):
        raise ImportError(
            f"{LIBRARY_PATH} is missing. Build it with "
            "`python -m losslessly_compressed_tensors_b200.build` (needs nvcc, targets sm_100a). "
            "There is no fallback implementation."
        )
    library = ctypes.CDLL(LIBRARY_PATH)
    for name, argtypes in _SIGNATURES.items():
        function = getattr(library, name)
        function.argtypes = argtypes
        function.restype = ctypes.c_int
    library.lct_version.restype = ctypes.c_char_p
    library.lct_error_string.restype = ctypes.c_char_p
    library.lct_error_string.argtypes = [ctypes.c_int]
    _library = library
    return library


def check(code: int, what: str) -> None:
    """Turn a non-zero return code of the library into an exception."""
    if code:
        text = load().lct_error_string(code).decode()
        raise RuntimeError(f"{what} failed: {text} (code {code})")
