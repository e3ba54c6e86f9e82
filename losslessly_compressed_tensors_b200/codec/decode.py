"""Host side of decoding: output allocation and the operand view for the decoder.

Follows ``LCT/codec/decode.py:18-92`` of the reference.  The overflow tails are
always substituted inside the decode launch; there is no second scatter pass.
"""
from __future__ import annotations

import torch

from ..comp_tensor import CompressedTensor
from ..compression.huffman_tables import get_distribution_tables
from ..kernels import dispatch
from ..kernels.backends import FallbackStorage


_OPERAND = "_b200_operand"   # per-object cache slot (not a field: outside equality and memory_size)


def _buffered(data: CompressedTensor) -> bool:
    return data.fallback_descriptor is not None


def _storage(data: CompressedTensor) -> FallbackStorage:
    """Overflow view of a compressed tensor: arena region or private tensors."""
    if _buffered(data):
        arena = data.fallback_buffer
        return FallbackStorage(
            tail=arena, count=data.fallback_count, lanes=arena, starts=arena,
            blocks=data.fallback_blocks, descriptor=data.fallback_descriptor,
            allocation=data.fallback_descriptor,
        )
    return FallbackStorage(
        tail=data.fallback_buffer, count=data.fallback_count,
        lanes=data.fallback_lanes, starts=data.fallback_starts,
        blocks=data.fallback_blocks, allocation=data.fallback_lanes,
        base=data.fallback_base,
    )


def has_fallback(data: CompressedTensor) -> bool:
    """True when the decoder has to consult overflow storage (always for buffered tensors,
    whose overflow count lives on the device)."""
    if data.layout != data.layout.COMPRESSED:
        return False
    if _buffered(data):
        return True
    return data.fallback_lanes is not None and data.fallback_lanes.numel() > 0


def operand_of(data: CompressedTensor):
    """The ``struct lct_operand`` describing ``data`` for the decoder and the fused operations.
    A compressed tensor is immutable, so the struct is built once and kept with it."""
    cached = data.__dict__.get(_OPERAND)
    if cached is not None:
        return cached
    device = data.data.device
    overflow = dispatch.fallback_tail_args(_storage(data) if has_fallback(data) else None)
    pair_table = dispatch.pair_table_for(data.distribution, device)
    shifted = data.decode_table
    if shifted is None:
        _, decode_table, _ = get_distribution_tables(data.distribution, device)
        shifted = dispatch.shift_decoding_table(decode_table, data.center)
    operand = dispatch.make_operand(data.data, data.sign_mantissa, shifted, data.center,
                                    pair_table, overflow)
    operand.keepalive = (shifted, pair_table)  # raw pointers inside: keep the tensors referenced
    object.__setattr__(data, _OPERAND, operand)
    return operand


def decode(data: CompressedTensor) -> torch.Tensor:
    """Decode to a BF16 tensor of the original shape."""
    logical_numel = data.logical_numel
    output = torch.empty(logical_numel, dtype=torch.int16, device=data.data.device)
    if logical_numel:
        _, _, rare_length = get_distribution_tables(data.distribution, data.data.device)
        block_symbols, lanes, steps, fixed_words = data.codec_geometry
        dispatch.decode_kernel(
            operand_of(data), output, data.size, logical_numel=logical_numel,
            block_symbols=block_symbols, lanes=lanes, steps=steps, fixed_words=fixed_words,
            rare_length=rare_length,
        )
    return output.view(torch.bfloat16).reshape(data.shape)


def decode_many(items: list[CompressedTensor]) -> list[torch.Tensor]:
    """Decode many compressed tensors with one launch per group of equal stream geometry and
    codebook family (one launch in all for the usual case of one codebook).  Same values as
    ``decode`` of each.  No counterpart in the reference (``LCT/codec/decode.py:60-92`` decodes
    one tensor per call)."""
    outputs: list[torch.Tensor | None] = [None] * len(items)
    groups: dict = {}
    for index, data in enumerate(items):
        if data.layout != data.layout.COMPRESSED:            # RAW: the dense source was kept
            outputs[index] = data.data.reshape(data.shape)
            continue
        device = data.data.device
        out = torch.empty(data.logical_numel, dtype=torch.int16, device=device)
        outputs[index] = out.view(torch.bfloat16).reshape(data.shape)
        if not data.logical_numel:
            continue
        _, _, rare_length = get_distribution_tables(data.distribution, device)
        groups.setdefault((device, data.codec_geometry, rare_length), []).append(
            (operand_of(data), out, data.size, data.logical_numel))
    for (device, stream_geometry, rare_length), jobs in groups.items():
        block_symbols, lanes, steps, fixed_words = stream_geometry
        dispatch.decode_batch(jobs, block_symbols=block_symbols, lanes=lanes, steps=steps,
                              fixed_words=fixed_words, rare_length=rare_length)
    return outputs
