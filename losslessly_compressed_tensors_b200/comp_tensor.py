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


def _owned_bytes(tensors) -> int:
    """Bytes of the distinct storages behind ``tensors`` (views of one storage count once)."""
    storages = {}
    for tensor in tensors:
        storage = tensor.untyped_storage()
        storages[(tensor.device, storage.data_ptr())] = storage.nbytes()
    return sum(storages.values())


@dataclass(frozen=True)
class CompressedTensor:
    """What ``compress`` returns.  The first three fields may be given positionally (as the
    reference's own constructor calls do); everything else is passed by keyword."""

    data: torch.Tensor                                # fixed payload words, or the dense source (RAW)
    size: int                                         # elements covered by codec storage, padding included
    sign_mantissa: torch.Tensor | None = None         # one side byte per storage position

    # -- what was compressed, and with which codebook -------------------------------------
    shape: tuple[int, ...] = ()
    layout: StorageLayout = StorageLayout.RAW
    distribution: Distribution = field(default_factory=Distribution)
    stream_geometry: tuple[int, int, int, int] | None = None
    center: torch.Tensor | int = 0                    # int32[1] sampled exponent center
    decode_table: torch.Tensor | None = None          # shifted first-level decode table, int32[1024]

    # -- overflow tails: counters and per-block metadata (both storage modes) ----------------
    fallback_count: torch.Tensor | None = None        # int32[1] number of overflow streams
    fallback_used: torch.Tensor | None = None         # int32[1] tail bytes
    fallback_blocks: torch.Tensor | None = None       # int32[3*blocks]: count | first entry | first byte

    # -- ... kept in private tensors of exact size -----------------------------------------------
    fallback_lanes: torch.Tensor | None = None        # storage lane per entry
    fallback_starts: torch.Tensor | None = None       # first overflow step per entry
    fallback_base: int = 0

    # -- ... or in a region of a shared arena ------------------------------------------------------
    buffer: TensorBuffer | None = None
    fallback_descriptor: torch.Tensor | None = None   # int32[4] arena descriptor
    fallback_buffer: torch.Tensor | None = None       # private tails, or the shared arena payload

    # -- constructor slots of older layouts, never set by this library -------------------------------
    offsets: torch.Tensor | None = None
    fallback_offsets: torch.Tensor | None = None

    @property
    def logical_numel(self) -> int:
        return math.prod(self.shape)

    @property
    def storage_numel(self) -> int:
        return self.size

    @property
    def codec_geometry(self) -> tuple[int, int, int, int]:
        """``(block_symbols, lanes, steps, fixed_words)`` this tensor was written with."""
        if self.layout is StorageLayout.COMPRESSED and self.fallback_blocks is None:
            raise ValueError("legacy compressed layout: decode with the original codec and recompress")
        if self.stream_geometry is not None:
            return self.stream_geometry
        from .codec.geometry import geometry

        clean_gaussian = (self.distribution.family is DistType.GAUSSIAN
                          and self.distribution.noise_level is NoiseLevel.CLEAN)
        # tensors written before the geometry was recorded used 24 words for that codebook
        return (65536, 256, 256, 24) if clean_gaussian else geometry(self.distribution)

    # -- memory ----------------------------------------------------------------------------------------

    def memory_buffer_size(self) -> int:
        """Bytes of the shared arena held by this tensor (0 when not buffered; one host sync)."""
        if self.fallback_descriptor is None:
            return 0
        return int(self.fallback_descriptor[1].item())

    def memory_size(self) -> int:
        """Device bytes owned by this tensor: every distinct tensor storage among its fields,
        and for a buffered tensor its arena region instead of the whole shared arena."""
        shared = self.fallback_descriptor is not None
        owned = [getattr(self, slot.name) for slot in fields(self)
                 if not (shared and slot.name == "fallback_buffer")]
        return (_owned_bytes(t for t in owned if isinstance(t, torch.Tensor))
                + self.memory_buffer_size())

    # -- leaving the process -------------------------------------------------------------------------

    def to_bytes(self) -> bytes:
        """Self-describing byte form (header with geometry, codebook, shape and component
        offsets, then the codec bytes); see ``serialization.py``.  One host synchronisation."""
        from .serialization import to_bytes

        return to_bytes(self)

    @classmethod
    def from_bytes(cls, blob, device="cuda") -> "CompressedTensor":
        """The tensor ``to_bytes`` wrote, on ``device``, owning all its memory."""
        from .serialization import from_bytes

        return from_bytes(blob, device)

    def free(self) -> None:
        """Return this tensor's arena region, if it has one.  Reading it afterwards is undefined."""
        if self.buffer is None or self.fallback_descriptor is None:
            return
        from .tensor_buffer import Allocation

        self.buffer.free(Allocation(self.fallback_descriptor, self.buffer))
