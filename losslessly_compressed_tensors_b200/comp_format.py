"""Codebook selector and storage-layout enums of the BF16 lossless codec.

Mirrors the public types of the reference's ``LCT/comp_format.py:6-74`` so that
user code written against ``LCT.comp_format`` keeps working: the same enum
members, the same ``Distribution`` fields, defaults, validation errors and
rounding rules (``param``/``mean`` snap to multiples of 0.25 with a 0.25 floor
on ``param``; ``zero_prob`` is clamped to [0, 1] and kept to two decimals).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass


class NoiseLevel(enum.Enum):
    """Fixed per-lane bit budget class (see ``codec.geometry``)."""

    CLEAN = 1
    MEDIUM = 2
    HIGH = 3
    SPARSE = 4


class DistType(enum.Enum):
    """Analytic family the exponent codebook is derived from."""

    EMPIRICAL = "empirical"
    GAUSSIAN = "gaussian"
    LAPLACE = "laplace"
    GAMMA = "gamma"


class StorageLayout(enum.Enum):
    """Whether a ``CompressedTensor`` holds codec streams or the dense source."""

    RAW = 1
    COMPRESSED = 2


_GRID = 0.25


def _finite(value: float, what: str) -> float:
    value = float(value)
    if not math.isfinite(value):
        raise ValueError(f"{what} must be finite")
    return value


@dataclass
class Distribution:
    """Selects the Huffman codebook (family, scale, location, zero mass) and the lane budget.

    ``param`` is the source scale (std for GAUSSIAN, scale otherwise), ``mean`` its
    location, ``zero_prob`` an added point mass at exact zero (``None`` = none).
    The tensor's actual scale is absorbed at encode time by the sampled exponent
    center, so ``param`` only shapes the code lengths.
    """

    family: DistType = DistType.EMPIRICAL
    param: float = 1.0
    mean: float = 0.0
    noise_level: NoiseLevel = NoiseLevel.CLEAN
    zero_prob: float | None = 0.0

    def __post_init__(self) -> None:
        if not isinstance(self.family, DistType):
            raise TypeError("family must be a DistType member")
        if not isinstance(self.noise_level, NoiseLevel):
            raise TypeError("noise_level must be a NoiseLevel member")
        scale = float(self.param)
        if not math.isfinite(scale) or scale <= 0.0:
            raise ValueError("distribution parameter must be finite and positive")
        location = _finite(self.mean, "distribution mean")
        zero = 0.0 if self.zero_prob is None else float(self.zero_prob)
        if not math.isfinite(zero) or zero < 0.0 or zero > 1.0:
            raise ValueError("zero_prob must be finite and between 0 and 1")
        # Snap to a coarse grid so the table cache stays small.
        self.param = float(max(_GRID, round(scale / _GRID) * _GRID))
        self.mean = float(round(location / _GRID) * _GRID)
        self.zero_prob = round(min(1.0, max(0.0, zero)), 2)

    def __str__(self) -> str:
        label = "std" if self.family is DistType.GAUSSIAN else "scale"
        return (
            f"{self.family.value}/{label}={self.param}/mean={self.mean}/"
            f"{self.noise_level.name.lower()}"
        )
