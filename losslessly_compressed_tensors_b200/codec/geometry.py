"""Stream geometry of the compressed format, per codebook family and noise level.

Same results as the reference's ``LCT/codec/geometry.py:13-39``.  A flattened
tensor is cut into blocks of ``block_symbols`` elements; a block is a
``steps x 256`` matrix whose 256 columns (lanes) are independent Huffman
streams with a fixed budget of ``fixed_words`` 32-bit words each.
"""
from __future__ import annotations

from ..comp_format import Distribution, DistType, NoiseLevel

LANES = 256

# (block_symbols, lane budget in bits) per layout; steps = block_symbols / 256.
_BIG, _SMALL = 65536, 32768
_LAYOUTS = {
    NoiseLevel.CLEAN: (_BIG, 800),                  # 3.125 bits per exponent
    NoiseLevel.SPARSE: (_BIG, 5 * (_BIG // LANES) // 2),   # 2.5 bits
    NoiseLevel.MEDIUM: (_SMALL, 800 - 6 * 32),      # 4.75 bits
    NoiseLevel.HIGH: (_SMALL, 800 - 3 * 32),        # 5.5 bits
}
# CLEAN + GAUSSIAN uses short blocks with exactly 3 bits per exponent.
_CLEAN_GAUSSIAN = (_SMALL, 3 * (_SMALL // LANES))


def geometry(distribution: Distribution) -> tuple[int, int, int, int]:
    """Return ``(block_symbols, lanes, steps, fixed_words)`` for newly written storage."""
    level = distribution.noise_level
    if level not in _LAYOUTS:
        raise ValueError(f"Unknown noise level: {level}")
    block_symbols, lane_bits = _LAYOUTS[level]
    if level is NoiseLevel.CLEAN and distribution.family is DistType.GAUSSIAN:
        block_symbols, lane_bits = _CLEAN_GAUSSIAN
    return block_symbols, LANES, block_symbols // LANES, lane_bits // 32
