"""Public functional API: lossless BF16 compression, decompression and fused updates.

Drop-in for the reference's ``LCT/operations.py:18-136``: same function names, argument names,
defaults and exceptions.  Everything here is routing; the work happens in ``codec/`` and, below
that, in the CUDA library.

    fused forms (A compressed, result dense or compressed):
        compA_add_B       A + B                      bf16 add
        compA_mul_B       A * B                      bf16 multiply
        a_compA_add_B     a*A + B                    fp32 fma, one rounding
        a_compA_add_b_B   a*A + b*B                  fp32 (B*b), fma, one rounding
        a_compA_add_compB a*A + B, both compressed   fp32 fma, one rounding
"""
from __future__ import annotations

import torch
from torch import Tensor

from .codec import decode as _decode, encode as _encode, pointwise as _pointwise
from .comp_format import Distribution, StorageLayout
from .comp_tensor import CompressedTensor
from .tensor_buffer import TensorBuffer


def _need_tensor(value, name: str) -> None:
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")


def _need_device_scalar(value, name: str, device: torch.device) -> None:
    _need_tensor(value, name)
    if value.numel() != 1 or value.dtype != torch.float32 or value.device != device:
        raise ValueError(f"{name} must be a float32 scalar on the compressed tensor's device")


def _need_matching_inner(A: Tensor, inner: int) -> None:
    if A.ndim != 2 or A.shape[1] != inner:
        raise ValueError("activation and weight inner dimensions must match")


def _dense_operand(A_comp, B, operation, where, **scalars):
    """All ``compA (op) dense B`` forms: ``where`` carries dense_output / buffer / distribution."""
    return _pointwise.pointwise_compressed_dense(A_comp, B, operation, **scalars, **where)


# ---- codec -------------------------------------------------------------------------------

@torch.compiler.disable
def compress(data: Tensor, distribution: Distribution | None = None,
             buffer: TensorBuffer | None = None, allow_raw: bool = False) -> CompressedTensor:
    """Losslessly encode the exponent bytes of a CUDA bfloat16 tensor (any shape).  With a
    ``buffer`` the overflow tails share its arena and nothing synchronises the host."""
    return _encode.encode(data.detach(), distribution if distribution is not None else Distribution(),
                          buffer, allow_raw=allow_raw)


@torch.compiler.disable
def decompress(data: CompressedTensor) -> Tensor:
    """The original tensor, bit for bit."""
    if data.layout != StorageLayout.COMPRESSED:      # RAW: the dense source was kept
        return data.data.reshape(data.shape)
    return _decode.decode(data)


@torch.compiler.disable
def compress_many(tensors: list[Tensor], distribution: Distribution | None = None,
                  buffer: TensorBuffer | None = None, *, recycle: bool = False) -> list[CompressedTensor]:
    """``compress`` of every tensor of a list with one codebook: four launches in all when a
    ``buffer`` is given (one call per tensor without one).  Same results, same arena.
    ``recycle``: reuse the storage of results released by ``free_many(..., recycle=True)``."""
    distribution = distribution if distribution is not None else Distribution()
    if buffer is None:
        return [compress(t, distribution, None) for t in tensors]
    return _encode.encode_many(list(tensors), distribution, buffer, recycle=recycle)


@torch.compiler.disable
def decompress_many(items: list[CompressedTensor]) -> list[Tensor]:
    """``decompress`` of every item with one launch per codebook geometry."""
    return _decode.decode_many(list(items))


def free_many(items: list[CompressedTensor], *, recycle: bool = False) -> None:
    """``free()`` of every item: one launch per arena instead of one per tensor, the regions
    returned in list order.  ``recycle``: the items' storage becomes available to later
    ``compress_many(..., recycle=True)`` calls; the items must not be used afterwards."""
    arenas: dict = {}
    for item in items:
        if item.buffer is not None and item.fallback_descriptor is not None:
            arenas.setdefault(id(item.buffer), (item.buffer, []))[1].append(item.fallback_descriptor)
    for buffer, descriptors in arenas.values():
        buffer.free_many(descriptors)
    if recycle:
        _encode.give_back(items)


# ---- matrix products through a decoded weight ----------------------------------------------

def A_compB(A: Tensor, B_comp: CompressedTensor) -> Tensor:
    """``A @ B_comp``."""
    _need_matching_inner(A, B_comp.shape[0])
    return A.contiguous() @ decompress(B_comp)


def A_compBT(A: Tensor, B_comp: CompressedTensor) -> Tensor:
    """``A @ B_comp.T``."""
    _need_matching_inner(A, B_comp.shape[1])
    return A.contiguous() @ decompress(B_comp).T


# ---- fused operations ------------------------------------------------------------------------

def compA_add_B(A_comp: CompressedTensor, B: Tensor, *, dense_output: bool = True,
                buffer: TensorBuffer | None = None, distribution=None):
    where = dict(dense_output=dense_output, buffer=buffer, distribution=distribution)
    return _dense_operand(A_comp, B, _pointwise.ADD, where)


def compA_mul_B(A_comp: CompressedTensor, B: Tensor, *, dense_output: bool = True,
                buffer: TensorBuffer | None = None, distribution=None):
    where = dict(dense_output=dense_output, buffer=buffer, distribution=distribution)
    return _dense_operand(A_comp, B, _pointwise.MULTIPLY, where)


def a_compA_add_B(A_comp: CompressedTensor, a: Tensor, B: Tensor, *, alpha_is_one: bool = False,
                  dense_output: bool = True, buffer: TensorBuffer | None = None,
                  distribution=None):
    """``alpha_is_one`` makes it ``A + B`` in fp32 without reading ``a``."""
    _need_tensor(a, "alpha")
    where = dict(dense_output=dense_output, buffer=buffer, distribution=distribution)
    return _dense_operand(A_comp, B, _pointwise.SCALAR_MUL_ADD, where, alpha=a,
                          alpha_is_one=alpha_is_one)


def a_compA_add_b_B(A_comp: CompressedTensor, a: Tensor, B: Tensor, b: Tensor, *,
                    alpha_is_one: bool = False, dense_output: bool = True,
                    buffer: TensorBuffer | None = None, distribution=None):
    """``B*b`` is rounded to fp32 first, then ``fma(A, a, .)``; with ``alpha_is_one`` the result
    is ``fma(B, b, A)``."""
    device = A_comp.data.device
    _need_device_scalar(a, "alpha", device)
    _need_device_scalar(b, "beta", device)
    where = dict(dense_output=dense_output, buffer=buffer, distribution=distribution)
    return _dense_operand(A_comp, B, _pointwise.SCALAR_MUL_ADD, where, alpha=a, beta=b,
                          alpha_is_one=alpha_is_one)


def a_compA_add_b_B_many(A_comps: list[CompressedTensor], a: Tensor, Bs: list[Tensor],
                         b: Tensor | None = None, *, alpha_is_one: bool = False,
                         buffer: TensorBuffer, distribution=None) -> list[CompressedTensor]:
    """``a * A + b * B`` (``b`` defaults to 1) for a whole list of compressed tensors of one
    codebook and geometry, results compressed into ``buffer``'s arena: five launches for the
    list instead of five per tensor, with the bytes ``a_compA_add_B`` / ``a_compA_add_b_B``
    (``dense_output=False``) give each tensor.  An optimizer's step over all its states.  No
    counterpart in the reference (``LCT/operations.py`` updates one tensor per call)."""
    device = A_comps[0].data.device
    if b is None:
        _need_tensor(a, "alpha")
    else:
        _need_device_scalar(a, "alpha", device)
        _need_device_scalar(b, "beta", device)
    return _pointwise.fused_update_many(A_comps, Bs, _pointwise.SCALAR_MUL_ADD, distribution,
                                        buffer, alpha=a, beta=b, alpha_is_one=alpha_is_one)


def a_compA_add_compB(A_comp: CompressedTensor, a: Tensor, B_comp: CompressedTensor, *,
                      dense_output: bool = True, buffer: TensorBuffer | None = None,
                      distribution=None):
    """Both operands decoded and combined in one launch."""
    _need_tensor(a, "alpha")
    return _pointwise.pointwise_scale_add_compressed(
        A_comp, B_comp, a, dense_output=dense_output, buffer=buffer, distribution=distribution)
