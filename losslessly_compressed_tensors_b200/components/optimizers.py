"""Optimizers that keep their BF16 state compressed between steps.

Drop-in for the three optimizers of the reference (``LCT/components/sparse_utils.py``:
``SparseSGDM`` :13-66, ``SparseMuon`` :98-160, ``SparseAdamW`` :163-214): same constructor
arguments, same update arithmetic in the same order, so a training script switches by
changing the import.  What differs is underneath: every update of compressed state runs
through this library's launch chains (``LCTTensor.mul_add_`` / ``lerp_`` / ``ema_square_``:
sample, center, decode -> arithmetic -> re-encode, scan, tails behind ONE library call;
``add_comp_``: both operands compressed), so the momentum of Muon and the moments of AdamW are
never decoded into a dense tensor of their own.

The codec is lossless, so wherever the compressed and the dense variant of an optimizer run
the same arithmetic on the dense values (Muon, AdamW) their trajectories are bit-identical;
``tests/test_gpu_optimizers.py`` checks exactly that.

Not taken over from the reference: the literal ``device="cuda"`` of its scalar tensors (the
parameters' device is used) and the tracing compiler around the Muon update (it runs eagerly).
"""
from __future__ import annotations

import math
from typing import Iterable

import torch
from torch import Tensor

from ..LCTensor import LCTTensor
from ..operations import a_compA_add_B
from ..tensor_buffer import TensorBuffer
from ..update_plan import UpdatePlan
from .dist_configs import momentum_dist, momentum_first_dist


def _scalar(value: float, like: Tensor) -> Tensor:
    return torch.tensor([value], dtype=torch.float32, device=like.device)


def _checked(params, *, matrices_only: bool = False) -> list:
    params = list(params)
    for p in params:
        if not isinstance(p, (LCTTensor, Tensor)):
            raise AssertionError("params must be a list of LCTTensor or Tensor")
        if matrices_only and p.ndim < 2:
            raise AssertionError("Muon requires matrix parameters")
    return params


class _Slot:
    """One piece of optimizer state: dense, or compressed while it is not being updated."""

    __slots__ = ("value",)

    def __init__(self):
        self.value: Tensor | LCTTensor | None = None

    def take_dense(self, like: Tensor, dtype: torch.dtype | None = None) -> Tensor:
        """The dense value (zeros shaped like ``like`` before the first step); a compressed one is
        decoded and its arena region released."""
        value, self.value = self.value, None
        if value is None:
            return torch.zeros_like(like, dtype=dtype)
        if isinstance(value, LCTTensor):
            return value.decompress_free()
        return value

    def put(self, dense: Tensor, *, compress: bool, buffer, dist) -> None:
        if compress and dense.dtype == torch.bfloat16:
            self.value = LCTTensor(dense, buffer=buffer, dist=dist)
        else:
            self.value = dense


class _Base:
    def _all_params(self):
        return self.params

    def zero_grad(self):
        for p in self._all_params():
            p.grad = None


class SparseSGDM(_Base):
    """``mom <- momentum * mom + g`` then ``p <- p - lr * mom``; with ``compressed`` the momentum
    never exists densely after its first step: both lines are fused kernels on the compressed
    state (fp32 fma, one rounding to BF16 each)."""

    def __init__(self, params: Iterable[LCTTensor | Tensor], lr, momentum=0.9,
                 buffer: TensorBuffer | None = None, compressed=True):
        self.params = _checked(params)
        self.lr, self.compressed, self.buffer = lr, compressed, buffer
        anchor = self.params[0] if self.params else torch.empty(0, device="cuda")
        self.momentum = torch.tensor(momentum, dtype=torch.float32, device=anchor.device)
        self.neg_lr = _scalar(-lr, anchor)
        self.momentums: list[Tensor | LCTTensor | None] = [None] * len(self.params)
        self._plan: UpdatePlan | None = None

    def _advance_momentum(self, index: int, grad: Tensor):
        state = self.momentums[index]
        if state is None:                      # first step: the gradient itself
            state = LCTTensor(grad, buffer=self.buffer, dist=momentum_dist) if self.compressed else grad
            self.momentums[index] = state
        elif self.compressed:
            state.mul_add_(self.momentum, grad)
        else:
            torch.add(grad, state, alpha=0.9, out=state)   # the reference's dense branch (literal 0.9)
        return state

    def _advance_all(self) -> bool:
        """From the second step on, with a shared arena: every momentum advanced by one prepared
        call for the whole parameter list (``UpdatePlan``: six launches per step, same values
        as one ``mul_add_`` each).  The momentum values alternate between the plan's two sets,
        so a reference to ``momentums[i].x`` is good for one more step only."""
        if not (self.compressed and self.buffer is not None and len(self.params) > 1
                and all(isinstance(m, LCTTensor) for m in self.momentums)):
            return False
        if self._plan is None:
            self._plan = UpdatePlan(self.momentums, self.momentum)
        self._plan.step([p.grad for p in self.params])
        return True

    @torch.no_grad()
    def step(self):
        advanced = self._advance_all()
        for index, p in enumerate(self.params):
            state = self.momentums[index] if advanced else self._advance_momentum(index, p.grad)
            if not self.compressed:
                p.add_(state * self.neg_lr)
            elif isinstance(p, LCTTensor):
                p.add_comp_(state, self.neg_lr)
            else:   # decode + fma in one kernel, written back into the same parameter storage
                p.copy_(a_compA_add_B(state.x, self.neg_lr, p))


def zeropower_via_newtonschulz5(G: Tensor, ns_iters: int) -> Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor, in BF16, with the
    coefficients (2, -1.5, 0.5) the reference uses (``sparse_utils.py:69-84``)."""
    assert G.ndim >= 2
    tall = G.size(-2) > G.size(-1)
    X = G.bfloat16().mT if tall else G.bfloat16()
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(ns_iters):
        gram = X @ X.mT
        X = 2 * X + (-1.5 * gram + 0.5 * gram @ gram) @ X
    return X.mT if tall else X


def _orthogonalised(direction: Tensor, ns_iters: int) -> Tensor:
    update = zeropower_via_newtonschulz5(direction, ns_iters)
    update *= max(1, direction.size(-2) / direction.size(-1)) ** 0.5
    return update


def muon_update(grad: Tensor, momentum: Tensor, mu=0.95, nesterov=True, ns_iters=5) -> Tensor:
    """In-place momentum step and the orthogonalised update (``sparse_utils.py:87-95``)."""
    momentum.lerp_(grad.to(momentum.dtype), 1 - mu)
    direction = grad.lerp_(momentum.to(grad.dtype), mu) if nesterov else momentum
    return _orthogonalised(direction, ns_iters)


def _fusable(state, grad: Tensor) -> bool:
    """Compressed state that the fused launch chains can update against ``grad`` directly."""
    return (isinstance(state, LCTTensor) and grad.dtype == torch.bfloat16
            and grad.is_contiguous() and state.x.buffer is not None)


class SparseMuon(_Base):
    """Muon with BF16 momentum kept compressed (the first step with the many-zeros codebook
    when ``zero_first_step``).  Momentum that lives in an arena is advanced by ONE launch chain
    on its compressed form - decode, ``lerp`` with the gradient, re-encode - which also writes
    the Nesterov direction over the gradient, so the dense momentum never exists; the values
    are those of the reference's decode / ``lerp_`` / ``lerp_`` / compress sequence
    (``sparse_utils.py:133-146``), which remains the route for everything else (first step,
    no arena, FP32 gradients)."""

    def __init__(self, params: Iterable[LCTTensor | Tensor], lr=0.02, weight_decay=0, mu=0.95,
                 buffer: TensorBuffer | None = None, compressed=True, distribution=None,
                 zero_first_step=False, ns_iters=5):
        self.params = _checked(params, matrices_only=True)
        self.lr, self.weight_decay, self.mu, self.ns_iters = lr, weight_decay, mu, ns_iters
        self.buffer, self.compressed = buffer, compressed
        self.distribution = distribution or momentum_dist
        self.first_step = zero_first_step
        anchor = self.params[0] if self.params else torch.empty(0, device="cuda")
        self.decay = _scalar(1 - lr * weight_decay, anchor)
        self.neg_lr = _scalar(-lr, anchor)
        self._momentum_weight = _scalar(1 - mu, anchor)     # lerp weights as float32, which is
        self._direction_weight = _scalar(mu, anchor)        # what torch's kernel makes of them
        self._slots = [_Slot() for _ in self.params]
        self._plan: UpdatePlan | None = None

    @property
    def momentums(self):
        return [slot.value for slot in self._slots]

    def _advance_all(self) -> bool:
        """Every momentum advanced by ONE prepared call for the whole parameter list (the
        momentum steps of different parameters are independent, so taking them out of the
        per-parameter loop changes no value): full waves of the fused kernel instead of one
        partial wave per tensor, six launches per step.  Needs every parameter to have a
        contiguous BF16 gradient and a momentum in this optimizer's arena, all of one shape
        class (one codebook, one geometry)."""
        states = [slot.value for slot in self._slots]
        grads = [p.grad for p in self.params]
        if not (self.compressed and not self.first_step and len(states) > 1
                and all(g is not None and _fusable(s, g) and s.x.buffer is self.buffer
                        and s.x.distribution == states[0].x.distribution
                        and s.x.codec_geometry == states[0].x.codec_geometry
                        and s.x.logical_numel for s, g in zip(states, grads))):
            return False
        if (self._plan is None or len(self._plan.tensors) != len(states)
                or any(a is not b for a, b in zip(self._plan.tensors, states))):
            from ..codec import pointwise
            from ..codec.geometry import geometry
            from ..kernels import dispatch
            if geometry(self.distribution) != states[0].x.codec_geometry:
                return False
            self._plan = UpdatePlan(states, self._momentum_weight, self._direction_weight,
                                    operation=pointwise.LERP, emit=dispatch.EMIT_NESTEROV,
                                    distribution=self.distribution)
        self._plan.step(grads, dense_outs=grads)
        return True

    @torch.no_grad()
    def step(self):
        advanced = self._advance_all()
        for slot, p in zip(self._slots, self.params):
            grad = p.grad
            if grad is None:
                continue
            dist = momentum_first_dist if self.first_step else self.distribution
            if advanced:
                update = _orthogonalised(grad, self.ns_iters)     # grad holds the direction now
            elif (self.compressed and _fusable(slot.value, grad)
                    and slot.value.x.buffer is self.buffer
                    and slot.value.lerp_(grad, self._momentum_weight, distribution=dist,
                                         nesterov_out=grad,
                                         nesterov_weight=self._direction_weight)):
                update = _orthogonalised(grad, self.ns_iters)
            else:
                momentum = slot.take_dense(grad, torch.bfloat16)
                update = muon_update(grad, momentum, mu=self.mu, ns_iters=self.ns_iters)
                slot.put(momentum, compress=self.compressed, buffer=self.buffer, dist=dist)
                del momentum
            if isinstance(p, LCTTensor):   # decay and update in one fused pass over the weights
                p.mul_add_(self.decay, update, beta=self.neg_lr, alpha_is_one=self.weight_decay == 0)
            else:
                p.mul_(1 - self.lr * self.weight_decay)
                p.add_(update, alpha=-self.lr)
        self.first_step = False


class SparseAdamW(_Base):
    """AdamW whose BF16 moments (and compressed matrix weights) are stored losslessly
    compressed; FP32 parameters and their moments stay dense.  Both modes run the same dense
    arithmetic on the decoded values."""

    def __init__(self, param_groups, *, betas=(0.8, 0.95), eps=1e-10, weight_decay=0,
                 compressed=True, buffer=None):
        self.param_groups = [dict(group, params=list(group["params"])) for group in param_groups]
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.compressed, self.buffer = compressed, buffer
        self.state: dict = {}
        self._device_scalars: dict = {}

    def _all_params(self):
        return [p for group in self.param_groups for p in group["params"]]

    def _update_one(self, p, grad: Tensor, lr: float) -> None:
        beta1, beta2 = self.betas
        state = self.state.setdefault(p, {"step": 0, "exp_avg": _Slot(), "exp_avg_sq": _Slot()})
        state["step"] += 1
        t = state["step"]
        first, second = state["exp_avg"], state["exp_avg_sq"]
        fused = (self.compressed and _fusable(first.value, grad) and _fusable(second.value, grad)
                 and first.value.x.buffer is self.buffer and second.value.x.buffer is self.buffer
                 and first.value.x.distribution == momentum_dist
                 and second.value.x.distribution == momentum_dist)
        if fused:
            # Both moments advance on their compressed forms; the dense new values that the
            # weight update reads are written by the same launches.
            scalars = self._scalars(grad)
            avg, square_avg = torch.empty_like(grad), torch.empty_like(grad)
            first.value.lerp_(grad, scalars[0], dense_out=avg)
            second.value.ema_square_(grad, scalars[1], scalars[2], dense_out=square_avg)
        else:
            avg = first.take_dense(grad)
            square_avg = second.take_dense(grad)
            avg.lerp_(grad, 1 - beta1)
            square_avg.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
        denom = square_avg.sqrt().div_(math.sqrt(1 - beta2 ** t)).add_(self.eps)
        weight = p.decompress() if isinstance(p, LCTTensor) else p
        weight.mul_(1 - lr * self.weight_decay)
        weight.addcdiv_(avg, denom, value=-lr / (1 - beta1 ** t))
        if isinstance(p, LCTTensor):
            previous = p.x
            p.x = LCTTensor(weight, buffer=previous.buffer, dist=previous.distribution).x
            previous.free()
        if not fused:
            for key, dense in (("exp_avg", avg), ("exp_avg_sq", square_avg)):
                state[key].put(dense, compress=self.compressed, buffer=self.buffer,
                               dist=momentum_dist)

    def _scalars(self, like: Tensor):
        """(1 - beta1, beta2, 1 - beta2) as float32 device scalars: the values PyTorch's kernels
        make of the Python numbers the reference passes."""
        key = like.device
        cached = self._device_scalars.get(key)
        if cached is None:
            beta1, beta2 = self.betas
            cached = self._device_scalars[key] = tuple(
                _scalar(v, like) for v in (1 - beta1, beta2, 1 - beta2))
        return cached

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    self._update_one(p, p.grad, group["lr"])
