"""``LCTTensor``: a tensor wrapper that keeps its values compressed.

Interface of the reference's ``LCT/LCTensor.py:12-111``: construction compresses, the
in-place updates replace the compressed value through the fused kernels and release the
previous value's arena region.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from .comp_format import Distribution
from .comp_tensor import CompressedTensor
from .operations import (
    a_compA_add_B, a_compA_add_b_B, a_compA_add_compB, compA_add_B, compress, decompress,
)
from .tensor_buffer import TensorBuffer


class LCTTensor(Tensor):
    __torch_function__ = torch._C._disabled_torch_function_impl
    x: CompressedTensor

    @staticmethod
    def __new__(cls, x, buffer: TensorBuffer | None, dist: Distribution):
        assert x.dtype == torch.bfloat16
        assert x.device.type == "cuda", f"x.device={x.device}"
        return torch.Tensor._make_wrapper_subclass(
            cls, x.shape, dtype=x.dtype, device=x.device, requires_grad=x.requires_grad)

    def __init__(self, x: Tensor, buffer: TensorBuffer | None, dist: Distribution):
        self.x = compress(x, buffer=buffer, distribution=dist)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        def dense(value):
            return decompress(value.x) if isinstance(value, LCTTensor) else value

        if func in (torch.ops.aten.t.default, torch.ops.aten.permute.default):
            return dense(args[0]).T
        if func is torch.ops.aten.mm.default:
            return dense(args[0]) @ dense(args[1])
        raise NotImplementedError(f"{func} not implemented for LCTTensor")

    @property
    def nbytes(self):
        return self.x.memory_size()

    @property
    def dense_nbytes(self):
        return math.prod(self.x.shape) * 2

    @property
    def layout(self):
        return "LCT compressed"

    def __repr__(self):
        return f"LCTTensor({self.x})"

    def _replace(self, new: CompressedTensor) -> None:
        previous, self.x = self.x, new
        previous.free()

    def add_(self, update: Tensor):
        """``x <- x + update``."""
        prev = self.x
        self._replace(compA_add_B(prev, update, dense_output=False,
                                  distribution=prev.distribution, buffer=prev.buffer))

    def mul_add_(self, alpha: Tensor, update: Tensor, beta: Tensor | None = None, *,
                 alpha_is_one: bool = False):
        """``x <- alpha * x + beta * update`` (``beta`` defaults to 1)."""
        prev = self.x
        common = dict(alpha_is_one=alpha_is_one, dense_output=False,
                      distribution=prev.distribution, buffer=prev.buffer)
        if beta is None:
            self._replace(a_compA_add_B(prev, alpha, update, **common))
        else:
            self._replace(a_compA_add_b_B(prev, alpha, update, beta, **common))

    def add_comp_(self, update_comp: "LCTTensor", alpha: Tensor):
        """``x <- x + alpha * update_comp`` with both sides compressed."""
        prev = self.x
        self._replace(a_compA_add_compB(update_comp.x, alpha, prev, dense_output=False,
                                        buffer=prev.buffer, distribution=prev.distribution))

    def decompress(self) -> Tensor:
        return decompress(self.x)

    def decompress_free(self) -> Tensor:
        """Decode, then release the compressed value's arena region."""
        dense = self.decompress()
        self.x.free()
        return dense

    def free(self):
        self.x.free()
