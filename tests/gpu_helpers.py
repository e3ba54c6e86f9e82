"""Helpers for the GPU parity tests: run the CUDA path, run the oracle, compare piece by piece."""
from __future__ import annotations

import numpy as np
import torch

from helpers import oracle_compress, region
from losslessly_compressed_tensors_b200.comp_tensor import CompressedTensor


def to_dev(bits: np.ndarray, device="cuda") -> torch.Tensor:
    """int16 BF16 bit patterns -> CUDA bfloat16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits).copy()).view(torch.bfloat16).to(device)


def bits_of(x: torch.Tensor) -> np.ndarray:
    return x.detach().contiguous().view(torch.int16).cpu().numpy().reshape(-1)


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def overflow_of(c: CompressedTensor):
    """(lanes, starts, tail) of a CUDA result as exact-size host arrays."""
    count = int(c.fallback_count.item())
    tail_bytes = int(c.fallback_used.item())
    if c.fallback_descriptor is None:
        return host(c.fallback_lanes), host(c.fallback_starts), host(c.fallback_buffer)
    base = int(c.fallback_descriptor[0].item())
    if base < 0:
        empty = np.zeros(0, np.uint8)
        return empty, empty, empty
    arena = host(c.fallback_buffer[base:base + 2 * count + tail_bytes])
    return arena[:count], arena[count:2 * count], arena[2 * count:]


def assert_same_components(c: CompressedTensor, want: dict, what: str = ""):
    """Every stored component of the CUDA result equals the oracle's, byte for byte."""
    assert int(c.center.item()) == want["center"], what
    assert tuple(c.stream_geometry) == tuple(want["geometry"]) and c.size == want["size"], what
    assert np.array_equal(host(c.decode_table), want["shifted_decode"]), what
    got_payload = host(c.data)
    assert got_payload.shape == want["encoded"].shape, what
    if not np.array_equal(got_payload, want["encoded"]):
        bad = np.nonzero(got_payload != want["encoded"])[0]
        raise AssertionError(f"{what}: {bad.size} payload words differ, first at {bad[:8]}")
    assert np.array_equal(host(c.sign_mantissa), want["side"]), what
    assert int(c.fallback_count.item()) == want["count"], what
    assert int(c.fallback_used.item()) == want["tail_bytes"], what
    assert np.array_equal(host(c.fallback_blocks), want["blocks"]), what
    lanes, starts, tail = overflow_of(c)
    if want["descriptor"] is None or want["descriptor"][2] == 0:
        assert np.array_equal(lanes, region(want, "lanes")), what
        assert np.array_equal(starts, region(want, "starts")), what
        assert np.array_equal(tail, region(want, "tail")), what
    if want["descriptor"] is not None:
        assert host(c.fallback_descriptor).tolist() == want["descriptor"].tolist(), what


def compress_both(oracle, bits: np.ndarray, dist, *, buffer=None, arena=None, shape=None):
    """Compress the same input with the CUDA path and the oracle."""
    from losslessly_compressed_tensors_b200.operations import compress

    x = to_dev(bits)
    if shape is not None:
        x = x.reshape(shape)
    got = compress(x, dist, buffer)
    want = oracle_compress(oracle, bits, dist, arena)
    return x, got, want
