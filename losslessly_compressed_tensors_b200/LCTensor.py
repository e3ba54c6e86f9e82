"""``LCTTensor``: a ``torch.Tensor`` wrapper subclass whose values live compressed.

Interface of the reference's ``LCT/LCTensor.py:12-111`` (constructor, ``x``, ``nbytes``,
``dense_nbytes``, ``layout``, ``add_``, ``mul_add_``, ``add_comp_``, ``decompress``,
``decompress_free``, ``free``; ``.T``/``permute``/``mm`` decode first).  Every in-place update
builds the new compressed value with one fused call on the old one, in the old value's codebook
and arena, and then returns the old value's arena region.  A value that an update replaced must
not be used again: besides its arena region, its storage is reused by a later update.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from . import operations as ops
from .codec import pointwise as _pointwise
from .comp_format import Distribution
from .comp_tensor import CompressedTensor
from .kernels import dispatch
from .tensor_buffer import TensorBuffer

_aten = torch.ops.aten


class LCTTensor(Tensor):
    __torch_function__ = torch._C._disabled_torch_function_impl
    x: CompressedTensor

    @staticmethod
    def __new__(cls, x, buffer: TensorBuffer | None, dist: Distribution):
        assert x.dtype == torch.bfloat16
        assert x.device.type == "cuda", f"x.device={x.device}"
        # shape / dtype / device / requires_grad of the wrapper follow the dense source
        return Tensor._make_wrapper_subclass(cls, x.shape, dtype=x.dtype, device=x.device,
                                             requires_grad=x.requires_grad)

    def __init__(self, x: Tensor, buffer: TensorBuffer | None, dist: Distribution):
        self.x = ops.compress(x, buffer=buffer, distribution=dist)

    # ---- the few aten ops the wrapper answers itself (by decoding) ------------------------

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        def dense(value):
            return ops.decompress(value.x) if isinstance(value, LCTTensor) else value

        if func in (_aten.t.default, _aten.permute.default):
            return dense(args[0]).T
        if func is _aten.mm.default:
            left, right = args
            return dense(left) @ dense(right)
        raise NotImplementedError(f"{func} not implemented for LCTTensor")

    # ---- sizes ---------------------------------------------------------------------------

    @property
    def nbytes(self):
        return self.x.memory_size()

    @property
    def dense_nbytes(self):
        return 2 * math.prod(self.x.shape)

    @property
    def layout(self):
        return "LCT compressed"

    def __repr__(self):
        return f"LCTTensor({self.x})"

    # ---- in-place updates ----------------------------------------------------------------

    def _become(self, make) -> None:
        """``make(old, home)`` builds the new value (``home``: compressed result in the old
        value's codebook and arena); the old value's region is released afterwards."""
        old = self.x
        home = dict(dense_output=False, distribution=old.distribution, buffer=old.buffer)
        self.x = make(old, home)
        old.free()

    def _update(self, update: Tensor, operation, **scalars) -> bool:
        """The update through recycled result storage (no allocation, one library call);
        False when that path does not apply to this value."""
        old = self.x
        new = _pointwise.recycled_update(old, update, operation, **scalars)
        if new is None:
            return False
        self.x = new        # `old` was released by the same call
        return True

    def add_(self, update: Tensor):
        """``x <- x + update``."""
        if not self._update(update, _pointwise.ADD):
            self._become(lambda old, home: ops.compA_add_B(old, update, **home))

    def mul_add_(self, alpha: Tensor, update: Tensor, beta: Tensor | None = None, *,
                 alpha_is_one: bool = False):
        """``x <- alpha * x + beta * update`` (``beta`` defaults to 1; ``alpha_is_one`` treats
        alpha as 1 without reading it)."""
        if beta is not None:
            ops._need_device_scalar(alpha, "alpha", self.x.data.device)
            ops._need_device_scalar(beta, "beta", self.x.data.device)
        else:
            ops._need_tensor(alpha, "alpha")
        if self._update(update, _pointwise.SCALAR_MUL_ADD, alpha=alpha, beta=beta,
                        alpha_is_one=alpha_is_one):
            return
        if beta is None:
            self._become(lambda old, home: ops.a_compA_add_B(
                old, alpha, update, alpha_is_one=alpha_is_one, **home))
        else:
            self._become(lambda old, home: ops.a_compA_add_b_B(
                old, alpha, update, beta, alpha_is_one=alpha_is_one, **home))

    def lerp_(self, end: Tensor, weight: Tensor, *, distribution: Distribution | None = None,
              nesterov_out: Tensor | None = None, nesterov_weight: Tensor | None = None,
              dense_out: Tensor | None = None) -> bool:
        """``x <- lerp(x, end, weight)`` with the arithmetic of ``torch.Tensor.lerp_`` on BF16
        CUDA tensors, as one launch chain on the compressed value: the momentum update of the
        reference's Muon and AdamW (``LCT/components/sparse_utils.py:88,193``) without the
        dense decoded state in between.  ``weight``: float32 device scalar.

        ``nesterov_out`` (with ``nesterov_weight``) also receives ``lerp(end, x_new,
        nesterov_weight)``, Muon's update direction (``sparse_utils.py:90``); it may be ``end``
        itself, which is how the reference computes it (``grad.lerp_``).  ``dense_out`` instead
        receives the new value densely.  ``distribution`` re-encodes with another codebook of
        the same geometry.

        Returns False, having done nothing, when the value is not in an arena or the codebooks'
        geometries differ: the caller then takes the decode / update / compress route."""
        if nesterov_out is not None and dense_out is not None:
            raise ValueError("one dense output at most")
        old = self.x
        emit = (dispatch.EMIT_NESTEROV if nesterov_out is not None
                else dispatch.EMIT_RESULT if dense_out is not None else dispatch.EMIT_NONE)
        new = _pointwise.recycled_update(
            old, end, _pointwise.LERP, alpha=weight, beta=nesterov_weight,
            distribution=distribution, emit=emit,
            dense_out=nesterov_out if nesterov_out is not None else dense_out)
        if new is None:
            return False
        self.x = new
        return True

    def ema_square_(self, grad: Tensor, decay: Tensor, weight: Tensor, *,
                    dense_out: Tensor | None = None) -> bool:
        """``x <- x.mul_(decay).addcmul_(grad, grad, value=weight)`` with PyTorch's BF16 CUDA
        arithmetic (two roundings), on the compressed value: AdamW's second moment
        (``sparse_utils.py:194``).  ``dense_out`` also receives the new value densely.  Returns
        False, having done nothing, when the value is not in an arena."""
        old = self.x
        new = _pointwise.recycled_update(
            old, grad, _pointwise.EMA_SQUARE, alpha=decay, beta=weight,
            emit=dispatch.EMIT_RESULT if dense_out is not None else dispatch.EMIT_NONE,
            dense_out=dense_out)
        if new is None:
            return False
        self.x = new
        return True

    @staticmethod
    def mul_add_many_(tensors: "list[LCTTensor]", alpha: Tensor, updates: "list[Tensor]",
                      beta: Tensor | None = None, *, alpha_is_one: bool = False,
                      group: int | None = 4) -> None:
        """``mul_add_`` of every tensor of the list with its own update, five launches per
        ``group`` tensors instead of five per tensor (all tensors must share the first one's
        codebook, geometry and arena).  Same values as calling ``mul_add_`` on each.  A group's
        old arena regions are released after all of its new ones have been reserved.  Groups
        let the host prepare the next call while the GPU works on the previous one;
        ``group=None`` puts the whole list into one call."""
        size = len(tensors) if not group else group
        for at in range(0, len(tensors), size):
            part = tensors[at:at + size]
            old = [tensor.x for tensor in part]
            new = ops.a_compA_add_b_B_many(old, alpha, updates[at:at + size], beta,
                                           alpha_is_one=alpha_is_one, buffer=old[0].buffer,
                                           distribution=old[0].distribution)
            for tensor, value, previous in zip(part, new, old):
                tensor.x = value
                previous.free()

    def add_comp_(self, update_comp: "LCTTensor", alpha: Tensor):
        """``x <- x + alpha * update_comp``, both sides compressed."""
        self._become(lambda old, home: ops.a_compA_add_compB(update_comp.x, alpha, old, **home))

    # ---- leaving the compressed form -------------------------------------------------------

    def decompress(self) -> Tensor:
        return ops.decompress(self.x)

    def decompress_free(self) -> Tensor:
        """The dense values; the compressed form's arena region is returned."""
        dense = self.decompress()
        self.free()
        return dense

    def free(self):
        self.x.free()
