"""Length-limited Huffman codebooks with one escape code, as two int32 tables.

Restates ``LCT/compression/huffman_tables.py:18-279`` of the reference so that
the tables (and therefore every compressed byte) are identical:

* code lengths by package-merge, at most 8 bits, ties resolved in favour of
  single symbols over packages and of the earlier symbol;
* the cheapest split of the 256 table indices into directly coded ones and
  ones sent as ``ESC + 8 literal bits`` (all splits are tried, the first best
  one wins);
* canonical codes, stored bit-reversed because the stream is filled LSB first;
* ``encode[index] = reversed_code | length << 20`` (int32[256]) and a first
  level decode table over ``FIRST_BITS`` = 10 stream bits,
  ``decode[prefix] = length | index << 8``, 0 under the escape prefix.

The tables are indexed by *table index* (0 = exact zero, else the centred
exponent delta); the kernels turn them into raw-exponent tables per tensor.
"""
from __future__ import annotations

from functools import lru_cache

import numpy as np
import torch

from ..comp_format import Distribution, DistType
from .probabilities import (
    _exponent_probabilities,
    empirical_probabilities,
    gamma_probabilities,
    gaussian_probabilities,
    laplace_probabilities,
)

FIRST_BITS = 10
FIRST_MASK = (1 << FIRST_BITS) - 1
_LITERAL_BITS = 8


def _length_limited_huffman_lengths(weights, max_length=FIRST_BITS):
    """Optimal prefix-code lengths with every length <= ``max_length`` (package-merge)."""
    weights = np.asarray(weights, dtype=np.longdouble)
    n = len(weights)
    if n == 0:
        return np.empty(0, dtype=np.int16)
    if np.any(weights < 0) or not np.any(weights > 0):
        raise ValueError("weights must be nonnegative and not all zero")
    if n > (1 << max_length):
        raise ValueError("Too many symbols for requested maximum length")
    if n <= 2:
        return np.ones(n, dtype=np.int16)

    order = np.argsort(weights, kind="stable")
    leaves = weights[order].tolist()

    # levels[d] lists, for merge level d+2, whether each item (ascending by
    # weight) is a package of two items of the level below.
    levels: list[list[bool]] = []
    below = leaves
    for _ in range(max_length - 1):
        pairs = [below[i] + below[i + 1] for i in range(0, len(below) - 1, 2)]
        merged: list = []
        flags: list[bool] = []
        li = pi = 0
        while li < n or pi < len(pairs):
            take_leaf = pi == len(pairs) or (li < n and leaves[li] <= pairs[pi])
            if take_leaf:
                merged.append(leaves[li])
                li += 1
            else:
                merged.append(pairs[pi])
                pi += 1
            flags.append(not take_leaf)
        levels.append(flags)
        below = merged

    # Walk back from the top level: the first `take` items of a level are in the
    # solution; every leaf among them deepens the next-lightest symbol by one,
    # every package pulls in two items of the level below.
    depth = np.zeros(n, dtype=np.int16)
    take = 2 * n - 2
    for flags in reversed(levels):
        chosen = flags[:take]
        packages = sum(chosen)
        depth[: len(chosen) - packages] += 1
        take = 2 * packages
    depth[:take] += 1

    lengths = np.empty(n, dtype=np.int16)
    lengths[order] = depth
    return lengths


def _optimal_escape_solution(probabilities, max_length=FIRST_BITS, max_esc_length=8):
    """Choose which table indices are coded directly and which go through ESC.

    With the indices sorted by falling probability, the ``k`` rarest share one
    ESC code followed by 8 literal bits.  Every ``k`` is costed exactly.
    """
    if max_esc_length is not None:
        max_length = min(max_length, max_esc_length)
    p = np.asarray(probabilities, dtype=np.longdouble)
    p /= p.sum()
    n = len(p)
    order = np.argsort(-p, kind="stable")
    ranked = p[order]
    rare_mass = np.zeros(n + 1, dtype=np.longdouble)
    rare_mass[1:] = np.cumsum(ranked[::-1], dtype=np.longdouble)

    lengths = _length_limited_huffman_lengths(ranked, max_length)
    best = {
        "cost": float(np.dot(ranked, lengths.astype(np.longdouble))),
        "k": 0, "lengths": lengths, "p_esc": 0.0,
    }
    for k in range(1, n):
        direct = n - k
        weights = np.empty(direct + 1, dtype=np.longdouble)
        weights[:direct] = ranked[:direct]
        weights[direct] = rare_mass[k]
        lengths = _length_limited_huffman_lengths(weights, max_length)
        cost = float(
            np.dot(weights, lengths.astype(np.longdouble)) + float(_LITERAL_BITS) * rare_mass[k]
        )
        if cost < best["cost"]:
            best = {"cost": cost, "k": k, "lengths": lengths.copy(), "p_esc": float(rare_mass[k])}

    k = best["k"]
    if k == 0:
        direct_indices, escaped_indices = order, np.empty(0, dtype=np.int64)
        direct_lengths, esc_length = best["lengths"], 0
    else:
        direct_indices, escaped_indices = order[: n - k], order[n - k:]
        direct_lengths, esc_length = best["lengths"][: n - k], int(best["lengths"][-1])
    return {
        "expected_bits": best["cost"],
        "k": k,
        "direct_indices": direct_indices,
        "escaped_indices": escaped_indices,
        "direct_lengths": direct_lengths,
        "esc_length": esc_length,
        "escape_probability": best["p_esc"],
    }


def _canonical_codes(lengths):
    """Canonical prefix codes ``{symbol: (code, length)}`` (MSB-first values)."""
    lengths = [int(v) for v in lengths]
    longest = max(lengths, default=0)
    per_length = [0] * (longest + 1)
    for length in lengths:
        per_length[length] += 1
    first = [0] * (longest + 1)
    code = 0
    for bits in range(1, longest + 1):
        code = (code + per_length[bits - 1]) << 1
        first[bits] = code
    codes = {}
    for symbol in sorted(range(len(lengths)), key=lambda s: (lengths[s], s)):
        length = lengths[symbol]
        codes[symbol] = (first[length], length)
        first[length] += 1
    return codes


def _reverse_bits(value: int, length: int) -> int:
    out = 0
    for _ in range(length):
        out = (out << 1) | (value & 1)
        value >>= 1
    return out


def _build_huffman_tables_from_lengths(probabilities, max_length=FIRST_BITS, max_esc_length=8):
    """Return ``(encode[256], decode[1 << FIRST_BITS], esc_length)`` as Python int lists."""
    solution = _optimal_escape_solution(
        probabilities, max_length=max_length, max_esc_length=max_esc_length,
    )
    direct = solution["direct_indices"]
    esc_length = solution["esc_length"]
    # ESC is one more symbol, placed after all direct ones.
    codes = _canonical_codes(np.concatenate([solution["direct_lengths"], [esc_length]]))
    esc_code = codes[len(direct)][0]

    words: dict[int, tuple[int, int]] = {}
    for position, index in enumerate(direct):
        words[int(index)] = codes[position]
    for index in solution["escaped_indices"]:
        index = int(index)
        literal = _reverse_bits(index & 255, _LITERAL_BITS)
        words[index] = ((esc_code << _LITERAL_BITS) | literal, esc_length + _LITERAL_BITS)

    encode = [0] * 256
    decode = [0] * (1 << FIRST_BITS)
    for index in range(256):
        code, length = words[index]
        encode[index] = _reverse_bits(code, length) | (length << 20)
    for index, (code, length) in words.items():
        lsb_first = _reverse_bits(code, length)
        if length > FIRST_BITS:
            decode[lsb_first & FIRST_MASK] = 0
            continue
        entry = length | (index << 8)
        for high in range(1 << (FIRST_BITS - length)):
            decode[lsb_first | (high << length)] = entry
    return encode, decode, esc_length


_FAMILY_PDF = {
    DistType.EMPIRICAL: lambda param, mean: empirical_probabilities(param, mean),
    DistType.GAUSSIAN: lambda param, mean: gaussian_probabilities(param, mean),
    DistType.LAPLACE: lambda param, mean: laplace_probabilities(param, mean),
    # The Gamma family is one fixed fit; param and mean do not enter.
    DistType.GAMMA: lambda param, mean: gamma_probabilities(),
}


@lru_cache(maxsize=None)
def host_tables(family: DistType, param: float, mean: float, zero_prob: float):
    """Cached host copy: ``(encode int32[256], decode int32[1024], rare_length)``."""
    if family not in _FAMILY_PDF:  # pragma: no cover - Distribution validates
        raise ValueError(f"unknown distribution family: {family!r}")
    probabilities = _exponent_probabilities(_FAMILY_PDF[family](param, mean), zero_prob)
    encode, decode, rare_length = _build_huffman_tables_from_lengths(
        probabilities, max_length=FIRST_BITS, max_esc_length=8,
    )
    encode = np.asarray(encode, dtype=np.int64).astype(np.int32)
    decode = np.asarray(decode, dtype=np.int64).astype(np.int32)
    encode.setflags(write=False)
    decode.setflags(write=False)
    return encode, decode, int(rare_length)


_device_tables: dict = {}


def get_distribution_tables(dist: Distribution, device=None):
    """Return ``(encode_table, decode_table, rare_length)`` as tensors on ``device``.

    The noise level does not enter.  ``device`` defaults to the current CUDA
    device; tables are cached per distribution and per device so that one
    process per GPU, or one process driving several GPUs, both work.
    """
    if not isinstance(dist, Distribution):
        raise TypeError("distribution must be a Distribution instance")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (dist.family, dist.param, dist.mean, dist.zero_prob, device)
    hit = _device_tables.get(key)
    if hit is None:
        encode, decode, rare_length = host_tables(*key[:4])
        hit = (
            torch.from_numpy(encode.copy()).to(device),
            torch.from_numpy(decode.copy()).to(device),
            rare_length,
        )
        _device_tables[key] = hit
    return hit
