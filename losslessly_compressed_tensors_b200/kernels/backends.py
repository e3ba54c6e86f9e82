"""The overflow-storage view handed from the host pipelines to the launch layer.

Same fields as the reference's ``FallbackStorage`` (``LCT/kernels/backends.py:36-50``).
The reference's backend table and GPU selection have no counterpart: there is
one set of sm_100a kernels.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class FallbackStorage:
    """Compact overflow metadata and its private or shared tail allocation."""

    tail: torch.Tensor
    count: torch.Tensor
    lanes: torch.Tensor
    starts: torch.Tensor
    blocks: torch.Tensor
    descriptor: torch.Tensor | None = None
    allocation: torch.Tensor | None = None
    base: int = 0

    @property
    def buffered(self) -> bool:
        return self.descriptor is not None
