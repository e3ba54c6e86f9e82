"""The immutable compressed form of one tensor.

Field for field the reference's ``CompressedTensor`` (``LCT/comp_tensor.py:12-96``),
so code that builds, inspects or frees one keeps working, and ``memory_size``
counts exactly the same set of allocations.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import TYPE_CHECKING

import torch

from .comp_format import Distribution, DistType, NoiseLevel, StorageLayout

if TYPE_CHECKING:
    from .tensor_buffer import TensorBuffer


@dataclass(frozen=True)
class CompressedTensor:
    data: torch.Tensor                                # fixed payload words, or the dense source (RAW)
    size: int                                         # elements covered by codec storage, padding included
    sign_mantissa: torch.Tensor | None = None         # one side byte per storage position
    offsets: torch.Tensor | None = None               # legacy slot, unused
    fallback_starts: torch.Tensor | None = None       # first overflow step per entry (private storage)
    fallback_offsets: torch.Tensor | None = None      # legacy slot, unused
    fallback_buffer: torch.Tensor | None = None       # private tails, or the shared arena payload
    fallback_descriptor: torch.Tensor | None = None   # int32[4] arena descriptor (buffered only)
    buffer: TensorBuffer | None = None
    fallback_base: int = 0
    fallback_count: torch.Tensor | None = None        # int32[1] number of overflow streams
    fallback_used: torch.Tensor | None = None         # int32[1] tail bytes
    distribution: Distribution = field(default_factory=Distribution)
    center: torch.Tensor | int = 0                    # int32[1] sampled exponent center
    shape: tuple[int, ...] = ()
    layout: StorageLayout = StorageLayout.RAW
    stream_geometry: tuple[int, int, int, int] | None = None
    fallback_lanes: torch.Tensor | None = None        # storage lane per entry (private storage)
    fallback_blocks: torch.Tensor | None = None       # int32[3*blocks]: count | first entry | first byte
    decode_table: torch.Tensor | None = None          # shifted first-level decode table, int32[1024]

    @property
    def codec_geometry(self) -> tuple[int, int, int, int]:
        """``(block_symbols, lanes, steps, fixed_words)`` this tensor was written with."""
        if self.layout is StorageLayout.COMPRESSED and self.fallback_blocks is None:
            raise ValueError("legacy compressed layout: decode with the original codec and recompress")
        if self.stream_geometry is not None:
            return self.stream_geometry
        from .codec.geometry import geometry

        legacy_gaussian = (
            self.distribution.family is DistType.GAUSSIAN
            and self.distribution.noise_level is NoiseLevel.CLEAN
        )
        return (65536, 256, 256, 24) if legacy_gaussian else geometry(self.distribution)

    def memory_size(self) -> int:
        """Device bytes owned by this tensor: every distinct tensor storage it holds, and for a
        buffered tensor its arena region (read from the descriptor: one host sync) instead of
        the whole shared arena."""
        buffered = self.fallback_descriptor is not None
        seen: dict[tuple[torch.device, int], int] = {}
        for slot in fields(self):
            value = getattr(self, slot.name)
            if not isinstance(value, torch.Tensor):
                continue
            if buffered and slot.name == "fallback_buffer":
                continue
            storage = value.untyped_storage()
            seen[(value.device, storage.data_ptr())] = storage.nbytes()
        total = sum(seen.values())
        if buffered:
            total += int(self.fallback_descriptor[1].item())
        return total

    def memory_buffer_size(self) -> int:
        """Bytes of the shared arena held by this tensor (0 when not buffered)."""
        if self.fallback_descriptor is None:
            return 0
        return int(self.fallback_descriptor[1].item())

    def free(self) -> None:
        """Return this tensor's arena region, if it has one.  Reading it afterwards is undefined."""
        if self.fallback_descriptor is None or self.buffer is None:
            return
        from .tensor_buffer import Allocation

        self.buffer.free(Allocation(self.fallback_descriptor, self.buffer))

    @property
    def logical_numel(self) -> int:
        return math.prod(self.shape)

    @property
    def storage_numel(self) -> int:
        return self.size
