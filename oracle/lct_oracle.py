"""ctypes front end of the CPU oracle (``lct_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg may
import this module, and only as the checker.  The shipped package never does.

The functions take and return NumPy arrays.  ``compress`` strings the C pieces
together in the order of the reference's host pipeline
(``LCT/codec/encode.py:22-186``) and returns every component of the
compressed form in a plain dict, so tests can compare them one by one.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liblct_oracle.so")

LANES = 256
OP_ADD, OP_MULTIPLY, OP_SCALED, OP_LERP, OP_EMA_SQUARE = 0, 1, 2, 3, 4


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the library is missing or stale."""
    src = os.path.join(_HERE, "lct_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.check_call(
            ["gcc", "-O2", "-fopenmp", "-fPIC", "-std=c11", "-ffp-contract=off", "-shared", "-o", _SO,
             src, "-lm"]
        )
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_estimate_center.restype = ctypes.c_int
        _lib.orc_buf_free.restype = ctypes.c_int
        _lib.orc_set_threads.restype = ctypes.c_int
    return _lib


def set_threads(n: int) -> int:
    """Use ``n`` host threads for the block loops (0 = leave as is); returns the count in use."""
    return int(lib().orc_set_threads(ctypes.c_int(n)))


def set_lane_mapping(name: str) -> None:
    """``"swizzle"`` (default) or ``"linear"``: the reference's ``config.lane_mapping``
    (``LCT/kernels/generic/layout.py:15-33``).  Process-wide, like the reference's setting."""
    if name not in ("swizzle", "linear"):
        raise ValueError(name)
    lib().orc_set_lane_mapping(ctypes.c_int(1 if name == "linear" else 0))


def _p(array):
    if array is None:
        return ctypes.c_void_p(0)
    assert array.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(array.ctypes.data)


_i64 = ctypes.c_int64
_i32 = ctypes.c_int


def estimate_center(src: np.ndarray, precomputed: bool = False) -> int:
    return int(lib().orc_estimate_center(_p(src), _i64(src.size), _i32(int(precomputed))))


def shift_tables(base_enc: np.ndarray, base_dec: np.ndarray, center: int):
    enc = np.empty(256, np.int32)
    dec = np.empty(1024, np.int32)
    lib().orc_shift_tables(_p(np.ascontiguousarray(base_enc, np.int32)),
                           _p(np.ascontiguousarray(base_dec, np.int32)), _i32(center), _p(enc), _p(dec))
    return enc, dec


def compress(src: np.ndarray, base_enc, base_dec, rare_length: int, geometry, *,
             precomputed: bool = False, side: np.ndarray | None = None, center: int | None = None,
             arena: dict | None = None) -> dict:
    """Encode ``src`` (int16 BF16 bits, or uint8 exponent bytes when ``precomputed``).

    ``arena``: ``None`` for private overflow storage, else a dict with ``meta``
    (int32 allocator words), ``regions`` and ``data`` (uint8 payload) that is
    updated in place like the reference's shared ``TensorBuffer``.
    """
    block_symbols, lanes, steps, fw = geometry
    assert lanes == LANES
    src = np.ascontiguousarray(src).reshape(-1)
    n = src.size
    blocks = -(-n // block_symbols)
    size = blocks * block_symbols
    streams = blocks * LANES
    if center is None:
        center = estimate_center(src, precomputed)
    enc, dec = shift_tables(base_enc, base_dec, center)
    encoded = np.zeros(streams * fw + 4, np.int32)
    defined = np.zeros(streams * fw + 4, np.uint8)
    if precomputed:
        assert side is not None and side.size == size
        side_defined = None
    else:
        side = np.zeros(size, np.uint8)
        side_defined = np.zeros(size, np.uint8)
    extra_starts = np.zeros(streams, np.uint8)
    summaries = np.zeros(4 * blocks, np.int32)
    lib().orc_encode(_p(src), _i32(int(precomputed)), _i64(n), _i64(size), _i32(block_symbols),
                     _i32(steps), _i32(fw), _p(enc), _p(side), _p(side_defined), _p(encoded),
                     _p(defined), _p(extra_starts), _p(summaries))
    counts = np.zeros(4, np.int32)
    lib().orc_prefix(_p(summaries), _i64(blocks), _p(counts))
    count, tail_bytes = int(counts[0]), int(counts[1])
    blocks_out = np.zeros(3 * blocks, np.int32)
    out = dict(
        geometry=tuple(geometry), logical_numel=n, size=size, center=center, rare_length=rare_length,
        shifted_encode=enc, shifted_decode=dec, encoded=encoded, defined=defined, side=side,
        side_defined=side_defined, extra_starts=extra_starts, summaries=summaries, counts=counts,
        blocks=blocks_out, count=count, tail_bytes=tail_bytes,
    )
    if arena is None:
        lanes_out = np.zeros(count, np.uint8)
        starts_out = np.zeros(count, np.uint8)
        tail = np.zeros(tail_bytes, np.uint8)
        offs = (0, 0, 0)
        descriptor = None
    else:
        descriptor = np.zeros(4, np.int32)
        buf_alloc(arena, tail_bytes, count, 2, descriptor)
        lanes_out = starts_out = tail = arena["data"]
        base = int(descriptor[0])
        offs = (base, base + count, base + 2 * count)
    if arena is None or descriptor[2] == 0 or count == 0:
        lib().orc_compact(_p(src), _i32(int(precomputed)), _i64(n), _i64(size), _i32(block_symbols),
                          _i32(steps), _p(extra_starts), _p(summaries), _p(lanes_out), _i64(offs[0]),
                          _p(starts_out), _i64(offs[1]), _p(tail), _i64(offs[2]), _p(blocks_out))
    out.update(lanes=lanes_out, starts=starts_out, tail=tail, offsets=offs, descriptor=descriptor)
    return out


def _overflow_args(c: dict):
    offs = c["offsets"]
    return (_p(c["blocks"]), _p(c["lanes"]), _i64(offs[0]), _p(c["starts"]), _i64(offs[1]),
            _p(c["tail"]), _i64(offs[2]))


def decompress(c: dict, *, plain: bool = False) -> np.ndarray:
    """Decode to int16 BF16 bits.  ``plain`` ignores the overflow storage."""
    block_symbols, _, steps, fw = c["geometry"]
    out = np.zeros(c["logical_numel"], np.int16)
    if c["logical_numel"] == 0:
        return out
    if plain:
        over = (_p(None), _p(None), _i64(0), _p(None), _i64(0), _p(None), _i64(0))
    else:
        over = _overflow_args(c)
    lib().orc_decode(_p(c["encoded"]), _p(c["side"]), _p(c["shifted_decode"]), _i32(c["center"]),
                     _i32(c["rare_length"]), _i64(c["logical_numel"]), _i64(c["size"]),
                     _i32(block_symbols), _i32(steps), _i32(fw), *over, _p(out))
    return out


def pointwise(c: dict, other: np.ndarray, op: int, alpha: float = 1.0, beta: float = 1.0, *,
              alpha_is_one: bool = True, beta_is_one: bool = True, dense: bool = True):
    """``compA (op) B``.  Returns BF16 bits (uint16) or ``(side, exponent_bytes)``."""
    block_symbols, _, steps, fw = c["geometry"]
    other = np.ascontiguousarray(other).reshape(-1).view(np.uint16)
    n, size = c["logical_numel"], c["size"]
    dense_out = np.zeros(n, np.uint16) if dense else None
    side_out = None if dense else np.zeros(size, np.uint8)
    exp_out = None if dense else np.zeros(size, np.uint8)
    lib().orc_pointwise(_p(c["encoded"]), _p(c["side"]), _p(c["shifted_decode"]), _i32(c["center"]),
                        _i32(c["rare_length"]), _i64(n), _i64(size), _i32(block_symbols), _i32(steps),
                        _i32(fw), *_overflow_args(c), _p(other), _i32(op), ctypes.c_float(alpha),
                        ctypes.c_float(beta), _i32(int(alpha_is_one)), _i32(int(beta_is_one)),
                        _p(dense_out), _p(side_out), _p(exp_out))
    return dense_out if dense else (side_out, exp_out)


def lerp_dense(start: np.ndarray, end: np.ndarray, weight: float) -> np.ndarray:
    """``bf16(torch.lerp(start, end, weight))`` on BF16 bit patterns, float32 arithmetic of
    PyTorch's CUDA kernel (``sparse_utils.py:90``: the Nesterov direction)."""
    start = np.ascontiguousarray(start).reshape(-1).view(np.uint16)
    end = np.ascontiguousarray(end).reshape(-1).view(np.uint16)
    out = np.zeros(start.size, np.uint16)
    lib().orc_lerp_dense(_p(start), _p(end), ctypes.c_float(weight), _i64(start.size), _p(out))
    return out


def dual(a: dict, b: dict, alpha: float, *, dense: bool = True):
    """``alpha * compA + compB`` for two operands of equal geometry."""
    block_symbols, _, steps, fw = a["geometry"]
    n, size = a["logical_numel"], a["size"]
    dense_out = np.zeros(n, np.uint16) if dense else None
    side_out = None if dense else np.zeros(size, np.uint8)
    exp_out = None if dense else np.zeros(size, np.uint8)

    def operand(c):
        return (_p(c["encoded"]), _p(c["side"]), _p(c["shifted_decode"]), _i32(c["center"]),
                *_overflow_args(c))

    lib().orc_dual(*operand(a), *operand(b), _i32(a["rare_length"]), _i64(n), _i64(size),
                   _i32(block_symbols), _i32(steps), _i32(fw), ctypes.c_float(alpha),
                   _p(dense_out), _p(side_out), _p(exp_out))
    return dense_out if dense else (side_out, exp_out)


# ---------------------------------------------------------------------------
# Arena allocator model
# ---------------------------------------------------------------------------

def new_arena(capacity: int, regions: int = 256) -> dict:
    arena = dict(meta=np.zeros(2 * regions + 3, np.int32), regions=regions,
                 data=np.zeros(capacity, np.uint8), capacity=capacity)
    lib().orc_buf_reset(_p(arena["meta"]), _i32(regions), _i32(capacity))
    return arena


def buf_reset(arena: dict) -> None:
    lib().orc_buf_reset(_p(arena["meta"]), _i32(arena["regions"]), _i32(arena["capacity"]))


def buf_alloc(arena: dict, nbytes: int, items: int = 0, item_bytes: int = 0,
              descriptor: np.ndarray | None = None, alignment: int = 16) -> np.ndarray:
    if descriptor is None:
        descriptor = np.zeros(4, np.int32)
    lib().orc_buf_alloc(_p(arena["meta"]), _i32(arena["regions"]), _i32(nbytes), _i32(items),
                        _i32(item_bytes), _i32(alignment), _p(descriptor))
    return descriptor


def buf_free(arena: dict, descriptor: np.ndarray) -> int:
    return int(lib().orc_buf_free(_p(arena["meta"]), _i32(arena["regions"]), _p(descriptor)))


def free_regions(arena: dict) -> list[tuple[int, int]]:
    r = arena["regions"]
    count = int(arena["meta"][2 * r])
    return [(int(arena["meta"][i]), int(arena["meta"][r + i])) for i in range(count)]


def memory_size(c: dict) -> int:
    """Bytes the reference's ``CompressedTensor.memory_size`` reports for this result
    (``LCT/comp_tensor.py:57-72``): payload, side bytes, block metadata, the
    4-int counts tensor, center, shifted decode table, plus private overflow
    tensors or the aligned arena allocation (and its 16-byte descriptor)."""
    blocks = c["size"] // c["geometry"][0]
    total = c["encoded"].nbytes + c["side"].nbytes + 12 * blocks + 16 + 4 + 4096
    if c["descriptor"] is None:
        total += 2 * c["count"] + c["tail_bytes"]
    else:
        total += 16 + int(c["descriptor"][1])
    return total
