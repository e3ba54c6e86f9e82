"""Public functional API: lossless BF16 compression, decompression and fused updates.

Same names, arguments and error behaviour as the reference's ``LCT/operations.py:18-136``.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .codec.decode import decode as decode_dense
from .codec.encode import encode as compress_dense
from .codec.pointwise import (
    ADD, MULTIPLY, SCALAR_MUL_ADD, pointwise_compressed_dense, pointwise_scale_add_compressed,
)
from .comp_format import Distribution, StorageLayout
from .comp_tensor import CompressedTensor
from .tensor_buffer import TensorBuffer


@torch.compiler.disable
def compress(data: Tensor, distribution: Distribution | None = None,
             buffer: TensorBuffer | None = None, allow_raw: bool = False) -> CompressedTensor:
    """Losslessly encode the exponent bytes of a CUDA bfloat16 tensor."""
    if distribution is None:
        distribution = Distribution()
    return compress_dense(data.detach(), distribution, buffer, allow_raw=allow_raw)


@torch.compiler.disable
def decompress(data: CompressedTensor) -> Tensor:
    """Decode a tensor produced by :func:`compress` (bit-exact)."""
    if data.layout == StorageLayout.COMPRESSED:
        return decode_dense(data)
    return data.data.reshape(data.shape)


def A_compBT(A: Tensor, B_comp: CompressedTensor) -> Tensor:
    """``A @ B_comp.T``."""
    if A.ndim != 2 or A.shape[1] != B_comp.shape[1]:
        raise ValueError("activation and weight inner dimensions must match")
    return A.contiguous() @ decompress(B_comp).T


def A_compB(A: Tensor, B_comp: CompressedTensor) -> Tensor:
    """``A @ B_comp``."""
    if A.ndim != 2 or A.shape[1] != B_comp.shape[0]:
        raise ValueError("activation and weight inner dimensions must match")
    return A.contiguous() @ decompress(B_comp)


def compA_add_B(A_comp: CompressedTensor, B: Tensor, *, dense_output: bool = True,
                buffer: TensorBuffer | None = None, distribution=None):
    """``A + B`` with A compressed."""
    return pointwise_compressed_dense(A_comp, B, ADD, dense_output=dense_output, buffer=buffer,
                                      distribution=distribution)


def compA_mul_B(A_comp: CompressedTensor, B: Tensor, *, dense_output: bool = True,
                buffer: TensorBuffer | None = None, distribution=None):
    """``A * B`` elementwise with A compressed."""
    return pointwise_compressed_dense(A_comp, B, MULTIPLY, dense_output=dense_output,
                                      buffer=buffer, distribution=distribution)


def a_compA_add_B(A_comp: CompressedTensor, a: Tensor, B: Tensor, *, alpha_is_one: bool = False,
                  dense_output: bool = True, buffer: TensorBuffer | None = None,
                  distribution=None):
    """``a * A + B`` (float32 fma, one rounding to BF16).  ``alpha_is_one`` skips reading ``a``."""
    if not isinstance(a, torch.Tensor):
        raise TypeError("alpha must be a torch.Tensor")
    return pointwise_compressed_dense(
        A_comp, B, SCALAR_MUL_ADD, alpha=a, alpha_is_one=alpha_is_one, dense_output=dense_output,
        buffer=buffer, distribution=distribution)


def a_compA_add_b_B(A_comp: CompressedTensor, a: Tensor, B: Tensor, b: Tensor, *,
                    alpha_is_one: bool = False, dense_output: bool = True,
                    buffer: TensorBuffer | None = None, distribution=None):
    """``a * A + b * B``: ``B * b`` rounded to float32, then ``fma(A, a, .)``, then BF16.
    With ``alpha_is_one`` the result is ``fma(B, b, A)``."""
    for name, scalar in (("alpha", a), ("beta", b)):
        if not isinstance(scalar, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if (scalar.numel() != 1 or scalar.dtype != torch.float32
                or scalar.device != A_comp.data.device):
            raise ValueError(
                f"{name} must be a float32 scalar on the compressed tensor's device")
    return pointwise_compressed_dense(
        A_comp, B, SCALAR_MUL_ADD, alpha=a, beta=b, alpha_is_one=alpha_is_one,
        dense_output=dense_output, buffer=buffer, distribution=distribution)


def a_compA_add_compB(A_comp: CompressedTensor, a: Tensor, B_comp: CompressedTensor, *,
                      dense_output: bool = True, buffer: TensorBuffer | None = None,
                      distribution=None):
    """``a * A + B`` with both operands compressed, decoded and combined in one launch."""
    if not isinstance(a, torch.Tensor):
        raise TypeError("alpha must be a torch.Tensor")
    return pointwise_scale_add_compressed(A_comp, B_comp, a, dense_output=dense_output,
                                          buffer=buffer, distribution=distribution)
