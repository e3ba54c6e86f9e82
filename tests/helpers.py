"""Helpers shared by the CPU and GPU tests."""
from __future__ import annotations

import numpy as np

from losslessly_compressed_tensors_b200.codec.geometry import geometry
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.compression.huffman_tables import host_tables
from synth import synth_bf16


def dist_of(spec: dict) -> Distribution:
    return Distribution(DistType[spec["family"]], param=spec.get("param", 1.0),
                        mean=spec.get("mean", 0.0), zero_prob=spec.get("zero_prob", 0.0),
                        noise_level=NoiseLevel[spec.get("noise", "CLEAN")])


def tables_of(dist: Distribution):
    return host_tables(dist.family, dist.param, dist.mean, dist.zero_prob)


def input_of(spec: dict) -> np.ndarray:
    return synth_bf16(spec["n"], spec["seed"], spec["kind"], spec.get("base", 0))


def oracle_compress(oracle, bits: np.ndarray, dist: Distribution, arena=None, **kwargs) -> dict:
    encode, decode, rare = tables_of(dist)
    return oracle.compress(bits, encode, decode, rare, geometry(dist), arena=arena, **kwargs)


def region(c: dict, what: str) -> np.ndarray:
    """lanes / starts / tail of an oracle result as exact-size arrays (private or arena)."""
    count, tail_bytes = c["count"], c["tail_bytes"]
    length = tail_bytes if what == "tail" else count
    offset = c["offsets"][{"lanes": 0, "starts": 1, "tail": 2}[what]]
    return np.asarray(c[what][offset:offset + length])
