"""Fused arithmetic on compressed tensors: ``compA (op) B`` and ``alpha * compA + compB``.

Interface of the reference's ``LCT/codec/pointwise.py:28-304``.  A fused launch decodes the
compressed operand(s), applies the operation with the reference's rounding (one BF16
rounding for add/multiply; float32 ``fma`` then round-to-nearest-even for the scaled forms)
and writes either dense BF16 or the split components, which then go through the normal
encode pipeline (new center sampled from the result).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from ..comp_format import Distribution, StorageLayout
from ..comp_tensor import CompressedTensor
from ..compression.huffman_tables import get_distribution_tables
from ..kernels import dispatch
from ..tensor_buffer import TensorBuffer
from . import encode as encode_module
from .decode import decode as decode_dense, operand_of
from .encode import encode as compress_dense, encode_components as compress_components
from .geometry import geometry


@dataclass(frozen=True)
class PointwiseOp:
    """An in-kernel operation code and the PyTorch expression with the same result."""

    name: str
    code: int
    torch_fn: object


ADD = PointwiseOp("add", dispatch.OP_ADD, torch.add)
MULTIPLY = PointwiseOp("multiply", dispatch.OP_MULTIPLY, torch.mul)
SCALAR_MUL_ADD = PointwiseOp(
    "scalar_mul_add", dispatch.OP_SCALAR_MUL_ADD,
    lambda left, right, alpha=1.0: (left.float() * alpha + right.float()).to(torch.bfloat16),
)
def _torch_ema_square(left, right, alpha, beta):
    return left.clone().mul_(float(alpha)).addcmul_(right, right, value=float(beta))


# The optimizers' state updates (``LCT/components/sparse_utils.py:88,193-194``); ``alpha`` is the
# lerp weight, resp. ``alpha`` = beta2 and ``beta`` = 1 - beta2 of the second-moment average.
LERP = PointwiseOp("lerp", dispatch.OP_LERP,
                   lambda left, right, alpha: torch.lerp(left, right, float(alpha)))
EMA_SQUARE = PointwiseOp("ema_square", dispatch.OP_EMA_SQUARE, _torch_ema_square)
POINTWISE_OPS = {op.name: op for op in (ADD, MULTIPLY, SCALAR_MUL_ADD, LERP, EMA_SQUARE)}


def _outputs(data: CompressedTensor, dense_output: bool):
    device = data.data.device
    if dense_output:
        output = torch.empty(data.logical_numel, dtype=torch.bfloat16, device=device)
        return output, output
    output = torch.empty(data.size, dtype=torch.uint8, device=device)
    return output, torch.empty_like(output)


def _scalar(value: Tensor | None, device) -> Tensor | None:
    if value is None:
        return None
    if value.dtype != torch.float32 or value.device != device:
        value = value.to(device=device, dtype=torch.float32)
    return value.reshape(-1)[:1].contiguous()


def _launch_pointwise_compressed_dense(data, other, operation, dense_output, *, alpha=None,
                                       beta=None, alpha_is_one=False):
    scaled = operation.name == "scalar_mul_add"
    device = data.data.device
    other = other.contiguous().view(-1)
    if other.dtype != torch.bfloat16:
        raise TypeError("the dense operand must be bfloat16")
    alpha = _scalar(alpha, device) if scaled and not alpha_is_one else None
    beta = _scalar(beta, device) if scaled else None
    _, _, rare_length = get_distribution_tables(data.distribution, device)
    block_symbols, lanes, steps, fixed_words = data.codec_geometry
    output, auxiliary = _outputs(data, dense_output)
    if data.logical_numel:
        dispatch.pointwise_dense(
            operand_of(data), other, output, auxiliary, data.size, alpha, beta,
            op=operation.code, alpha_is_one=not scaled or alpha_is_one,
            beta_is_one=not scaled or beta is None, compressed_output=not dense_output,
            rare_length=rare_length, logical_numel=data.logical_numel,
            block_symbols=block_symbols, lanes=lanes, steps=steps, fixed_words=fixed_words,
        )
    return output, auxiliary


# The compressed-output forms of ``compA (op) B`` run as one fused launch (decode, operate,
# re-encode) after a small pre-pass that samples the result's center.  Setting this to False
# restores the reference's two-stage order (split intermediate, then the encoder); the results
# are bit-identical either way.
FUSED_UPDATE = True


_SAMPLE_VALUES = "_b200_sample_values"   # attribute of a CompressedTensor made by a fused update


def _fused_update(data, other, operation, result_distribution, buffer, *, alpha, beta,
                  alpha_is_one):
    scaled = operation.name == "scalar_mul_add"
    device = data.data.device
    other = other.contiguous().view(-1)
    if other.dtype != torch.bfloat16:
        raise TypeError("the dense operand must be bfloat16")
    alpha = _scalar(alpha, device) if scaled and not alpha_is_one else None
    beta = _scalar(beta, device) if scaled else None
    _, _, rare_length = get_distribution_tables(data.distribution, device)
    block_symbols, lanes, steps, fixed_words = data.codec_geometry
    operand = operand_of(data)
    meta = dict(op=operation.code, alpha_is_one=not scaled or alpha_is_one,
                beta_is_one=not scaled or beta is None, rare_length=rare_length,
                logical_numel=data.logical_numel, block_symbols=block_symbols, lanes=lanes,
                steps=steps, fixed_words=fixed_words)
    count = min(data.logical_numel, 4096)
    samples = torch.empty(count, dtype=torch.uint8, device=device)
    # The BF16 results at the sample positions ride along with the result (outside the
    # reference's field set and its memory_size()): when the result is updated again, they
    # replace the walk over its bit streams in the sample pre-pass.
    known = getattr(data, _SAMPLE_VALUES, None)
    if known is not None and (known.numel() != count or known.device != device):
        known = None
    values = torch.empty(count, dtype=torch.int16, device=device)
    meta_sample = dict(meta, known_values=known, result_values=values)
    side_out = torch.empty(data.size, dtype=torch.uint8, device=device)
    spill = torch.empty(data.size, dtype=torch.uint8, device=device)  # touched by overflow lanes only
    if buffer is not None and encode_module.SINGLE_CALL_PIPELINE:
        # One call for the whole update; same launches and bytes as the staged sequence below.
        if buffer.capacity_bytes % 4:
            raise ValueError("TensorBuffer capacity must be divisible by 4")
        encode_table, decode_table, _ = get_distribution_tables(result_distribution, device)
        blocks = data.size // block_symbols
        streams = blocks * lanes

        def new(n, dtype):
            return torch.empty(n, dtype=dtype, device=device)

        center, counts, descriptor = new(1, torch.int32), new(4, torch.int32), new(4, torch.int32)
        shifted_decode = new(decode_table.numel(), torch.int32)
        encoded = new(streams * fixed_words + 4, torch.int32)
        blocks_out = new(3 * blocks, torch.int32)
        dispatch.update_pipeline(
            operand, other, alpha, beta, encode_table, decode_table, samples, center,
            new(256, torch.int32), shifted_decode, side_out, encoded, new(streams, torch.uint8),
            new(4 * blocks, torch.int32), spill, counts, descriptor, blocks_out, buffer, data.size,
            **meta_sample)
        result = CompressedTensor(
            encoded, data.size, side_out, fallback_starts=None, fallback_lanes=None,
            fallback_blocks=blocks_out, fallback_buffer=buffer.data,
            fallback_descriptor=descriptor, buffer=buffer, fallback_count=counts[:1],
            fallback_used=counts[1:2], distribution=result_distribution, center=center,
            decode_table=shifted_decode, shape=data.shape, layout=StorageLayout.COMPRESSED,
            stream_geometry=geometry(result_distribution),
        )
        object.__setattr__(result, _SAMPLE_VALUES, values)
        return result
    dispatch.update_sample(operand, other, samples, data.size, alpha, beta, **meta_sample)

    def launch(shifted_encode, encoded, extra_starts, summaries):
        dispatch.update_fused(operand, other, shifted_encode, side_out, encoded, extra_starts,
                              summaries, spill, data.size, alpha, beta, **meta)

    result = compress_components(
        spill, side_out, data.size, result_distribution, buffer, data.shape, precomputed=True,
        logical_numel=data.logical_numel, center_samples=samples, launch_encode=launch,
    )
    object.__setattr__(result, _SAMPLE_VALUES, values)
    return result


# ---------------------------------------------------------------------------
# In-place updates with recycled result storage
# ---------------------------------------------------------------------------
#
# ``LCTTensor.mul_add_`` / ``add_`` replace a value by a new one and release the old one at
# once.  Going through ``_fused_update`` that costs about a dozen small allocations, a dataclass
# and an operand record per call - more host time than the GPU needs for a 16 Mi-element
# tensor.  Here the storage of a released value is kept (per stream, arena, codebook and shape)
# and becomes the next result of the same kind, together with the C arguments that describe
# it, so a call is ONE library call of four launches (sample + center, decode -> op -> encode,
# scan + reservation + release of the old region, tails) and no allocation.  Twelve momentum tensors of one shape share ONE spare set: memory grows
# by one compressed tensor per shape, not per tensor.

_RESULT_SET = "_b200_result_set"    # attribute of a CompressedTensor whose storage may be reused
MAX_SPARE_SETS = 2                  # spare result sets kept per kind
MAX_KINDS = 32                      # kinds whose work buffers and spare sets are kept


def forget_spare_storage() -> None:
    """Drop every spare result set and work buffer held for ``LCTTensor`` updates."""
    _kinds.clear()


class _ResultSet:
    """Storage of one fused-update result and the C arguments that point into it."""

    __slots__ = ("value", "middle", "outputs", "tail", "kind")


class _Kind:
    """Everything updates of one (stream, arena, codebook, shape) share: tables, work buffers
    (reused by every call: calls on one stream run in order, and the first launch of an update
    is an ordinary launch that waits for all earlier work) and the spare result sets."""

    def __init__(self, data: CompressedTensor, result_distribution, buffer):
        if buffer.capacity_bytes % 4:
            raise ValueError("TensorBuffer capacity must be divisible by 4")
        device = data.data.device
        self.device, self.buffer, self.distribution = device, buffer, result_distribution
        self.shape, self.size, self.logical_numel = data.shape, data.size, data.logical_numel
        self.geometry = block_symbols, lanes, steps, fixed_words = data.codec_geometry
        self.encode_table, self.decode_table, _ = get_distribution_tables(result_distribution, device)
        _, _, self.rare_length = get_distribution_tables(data.distribution, device)
        self.blocks = data.size // block_symbols
        self.count = min(data.logical_numel, 4096)

        self.samples = self._new(self.count, torch.uint8)
        self.shifted_encode = self._new(256, torch.int32)
        self.extra_starts = self._new(self.blocks * lanes, torch.uint8)
        self.summaries = self._new(4 * self.blocks, torch.int32)
        self.spill = self._new(data.size, torch.uint8)
        self.release_status = self._new(1, torch.int32)
        self.head = (self.encode_table.data_ptr(), self.decode_table.data_ptr(),
                     self.samples.data_ptr())
        self.work = (self.extra_starts.data_ptr(), self.summaries.data_ptr(), self.spill.data_ptr())
        self.rest = (buffer._storage.data_ptr(), buffer.max_free_regions, data.size,
                     data.logical_numel, block_symbols, steps, fixed_words, self.rare_length)
        self.spare: list[_ResultSet] = []

    def _new(self, count, dtype):
        return torch.empty(count, dtype=dtype, device=self.device)

    def take(self) -> _ResultSet:
        if self.spare:
            return self.spare.pop()
        new = self._new
        _, lanes, _, fixed_words = self.geometry
        counts, descriptor = new(4, torch.int32), new(4, torch.int32)
        center, values = new(1, torch.int32), new(self.count, torch.int16)
        shifted_decode = new(self.decode_table.numel(), torch.int32)
        encoded = new(self.blocks * lanes * fixed_words + 4, torch.int32)
        side, blocks_out = new(self.size, torch.uint8), new(3 * self.blocks, torch.int32)
        value = CompressedTensor(
            encoded, self.size, side, fallback_starts=None, fallback_lanes=None,
            fallback_blocks=blocks_out, fallback_buffer=self.buffer.data,
            fallback_descriptor=descriptor, buffer=self.buffer, fallback_count=counts[:1],
            fallback_used=counts[1:2], distribution=self.distribution, center=center,
            decode_table=shifted_decode, shape=self.shape, layout=StorageLayout.COMPRESSED,
            stream_geometry=geometry(self.distribution),
        )
        object.__setattr__(value, _SAMPLE_VALUES, values)
        result = _ResultSet()
        result.value, result.kind = value, self
        result.middle = (values.data_ptr(), center.data_ptr())
        result.outputs = (shifted_decode.data_ptr(), side.data_ptr(), encoded.data_ptr())
        result.tail = (counts.data_ptr(), descriptor.data_ptr(), blocks_out.data_ptr())
        object.__setattr__(value, _RESULT_SET, result)
        return result


_kinds: dict = {}


def recycled_update(data: CompressedTensor, other: Tensor, operation: PointwiseOp, *,
                    alpha: Tensor | None = None, beta: Tensor | None = None,
                    alpha_is_one: bool = False, distribution: Distribution | None = None,
                    emit: int = dispatch.EMIT_NONE,
                    dense_out: Tensor | None = None) -> CompressedTensor | None:
    """The in-place update ``data <- data (op) other``: returns the new value, compressed into
    ``data``'s arena with ``distribution``'s codebook (default: ``data``'s own) in storage
    recycled from an earlier result, and releases ``data`` in the same call - its arena region
    goes back right after the new one has been reserved, and its storage becomes the spare set
    of a later update.  ``data`` must not be used afterwards.  ``emit`` / ``dense_out``: also write the dense result
    (``EMIT_RESULT``) or the Nesterov direction ``lerp(other, result, beta)`` (``EMIT_NESTEROV``,
    ``LERP`` only) to ``dense_out``, a contiguous BF16 tensor of ``data``'s shape that may be
    ``other`` itself.  Returns ``None`` when this path does not apply (no arena, RAW or empty
    tensor, staged pipeline, a result codebook of another geometry)."""
    buffer = data.buffer
    result_distribution = distribution or data.distribution
    if (buffer is None or data.layout != StorageLayout.COMPRESSED or not data.logical_numel
            or not FUSED_UPDATE or not encode_module.SINGLE_CALL_PIPELINE
            or geometry(result_distribution) != data.codec_geometry):
        return None
    if tuple(other.shape) != data.shape:
        raise ValueError(f"{operation.name} expects tensors with the same shape")
    if other.dtype != torch.bfloat16:
        raise TypeError("the dense operand must be bfloat16")
    if not other.is_contiguous():
        other = other.contiguous()
    device = data.data.device
    scaled = operation is SCALAR_MUL_ADD
    takes_scalars = scaled or operation is LERP or operation is EMA_SQUARE
    if takes_scalars and alpha is None and not (scaled and alpha_is_one):
        raise ValueError(f"{operation.name} requires an alpha argument")
    if operation is EMA_SQUARE and beta is None:
        raise ValueError("ema_square requires a beta argument")
    alpha = _scalar(alpha, device) if takes_scalars and not (scaled and alpha_is_one) else None
    beta = _scalar(beta, device) if takes_scalars else None
    if emit != dispatch.EMIT_NONE:
        if (dense_out is None or dense_out.dtype != torch.bfloat16 or dense_out.device != device
                or tuple(dense_out.shape) != data.shape or not dense_out.is_contiguous()):
            raise ValueError("dense_out must be a contiguous bfloat16 tensor of the operand's "
                             "shape on its device")
        if emit == dispatch.EMIT_NESTEROV and (operation is not LERP or beta is None):
            raise ValueError("the Nesterov direction needs the lerp operation and its weight (beta)")
    index = device.index if device.index is not None else torch.cuda.current_device()
    d, r = data.distribution, result_distribution
    key = (index, dispatch._raw_stream(index), id(buffer), d.family, d.param, d.mean, d.zero_prob,
           r.family, r.param, r.mean, r.zero_prob, r.noise_level, data.shape, data.logical_numel)
    kind = _kinds.pop(key, None)
    if kind is None or kind.buffer is not buffer:
        kind = _Kind(data, result_distribution, buffer)
    _kinds[key] = kind                       # most recently used last
    while len(_kinds) > MAX_KINDS:
        _kinds.pop(next(iter(_kinds)))
    target = kind.take()
    known = data.__dict__.get(_SAMPLE_VALUES)
    if known is not None and (known.numel() != kind.count or known.device != device):
        known = None
    dispatch._call(
        "lct_update_emit", device,
        dispatch.ctypes.byref(operand_of(data)), other.data_ptr(),
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        operation.code, int(not scaled or alpha_is_one), int(not scaled or beta is None),
        *kind.head, known.data_ptr() if known is not None else None, *target.middle,
        kind.shifted_encode.data_ptr(), *target.outputs, *kind.work, *target.tail, *kind.rest,
        dense_out.data_ptr() if emit != dispatch.EMIT_NONE else None, emit,
        data.fallback_descriptor.data_ptr(), kind.release_status.data_ptr(),
        launches=4 if known is not None else 5)
    held = data.__dict__.get(_RESULT_SET)
    if held is not None and len(held.kind.spare) < MAX_SPARE_SETS:
        held.kind.spare.append(held)
    return target.value


def fused_update_many(datas, others, operation, result_distribution, buffer, *, alpha=None,
                      beta=None, alpha_is_one=False):
    """``_fused_update`` of many compressed tensors in five launches in all: every tensor of
    ``datas`` (one codebook, one geometry, one device, none RAW or empty) is combined with its
    dense partner in ``others`` and re-encoded into ``buffer``'s arena.  Each result holds the
    bytes the one-tensor call gives it; the arena reservations are made in list order."""
    if not datas or len(datas) != len(others):
        raise ValueError("fused_update_many needs as many dense operands as compressed tensors")
    if buffer is None or buffer.capacity_bytes % 4:
        raise ValueError("fused_update_many needs a TensorBuffer whose capacity is divisible by 4")
    first = datas[0]
    device = first.data.device
    scaled = operation.name == "scalar_mul_add"
    if scaled and alpha is None:
        raise ValueError("scalar_mul_add requires an alpha argument")
    result_distribution = result_distribution or first.distribution
    block_symbols, lanes, steps, fixed_words = first.codec_geometry
    if geometry(result_distribution) != first.codec_geometry:
        raise ValueError("matrix compressed output must preserve the input stream geometry")
    alpha = _scalar(alpha, device) if scaled and not alpha_is_one else None
    beta = _scalar(beta, device) if scaled else None
    encode_table, decode_table, rare_length = get_distribution_tables(result_distribution, device)
    flat = []
    for data, other in zip(datas, others):
        if (data.layout != StorageLayout.COMPRESSED or data.distribution != first.distribution
                or data.codec_geometry != first.codec_geometry or data.data.device != device
                or not data.logical_numel):
            raise ValueError("fused_update_many needs non-empty compressed tensors of one codebook, "
                             "geometry and device")
        if tuple(other.shape) != data.shape:
            raise ValueError(f"{operation.name} expects tensors with the same shape")
        other = other.contiguous().view(-1)
        if other.dtype != torch.bfloat16:
            raise TypeError("the dense operand must be bfloat16")
        flat.append(other)
    # Every result owns its tensors (memory_size() counts storages); only the spill arrays,
    # which nothing reads after the call, share one allocation (sizes are multiples of the
    # 32768-element block, so every slice starts on a 16-byte boundary).
    def new(count, dtype):
        return torch.empty(count, dtype=dtype, device=device)

    spill_pool = new(sum(d.size for d in datas), torch.uint8)
    jobs, results = [], []
    at = 0
    for data, other in zip(datas, flat):
        blocks = data.size // block_symbols
        count = min(data.logical_numel, 4096)
        center, counts, descriptor = new(1, torch.int32), new(4, torch.int32), new(4, torch.int32)
        shifted_decode = new(decode_table.numel(), torch.int32)
        blocks_out = new(3 * blocks, torch.int32)
        side_out = new(data.size, torch.uint8)
        encoded = new(blocks * lanes * fixed_words + 4, torch.int32)
        values = new(count, torch.int16)
        known = getattr(data, _SAMPLE_VALUES, None)
        if known is not None and (known.numel() != count or known.device != device):
            known = None
        jobs.append(dict(operand=operand_of(data), other=other, known_values=known,
                         result_values=values, side_out=side_out, encoded_out=encoded,
                         spill=spill_pool[at:at + data.size], center=center,
                         decode_table=shifted_decode, counts=counts, descriptor=descriptor,
                         blocks=blocks_out, size=data.size, logical_numel=data.logical_numel))
        result = CompressedTensor(
            encoded, data.size, side_out, fallback_starts=None, fallback_lanes=None,
            fallback_blocks=blocks_out, fallback_buffer=buffer.data,
            fallback_descriptor=descriptor, buffer=buffer, fallback_count=counts[:1],
            fallback_used=counts[1:2], distribution=result_distribution, center=center,
            decode_table=shifted_decode, shape=data.shape, layout=StorageLayout.COMPRESSED,
            stream_geometry=geometry(result_distribution),
        )
        object.__setattr__(result, _SAMPLE_VALUES, values)
        results.append(result)
        at += data.size
    dispatch.update_batch(
        jobs, alpha, beta, encode_table, decode_table, buffer, op=operation.code,
        alpha_is_one=not scaled or alpha_is_one, beta_is_one=not scaled or beta is None,
        rare_length=rare_length, block_symbols=block_symbols, lanes=lanes, steps=steps,
        fixed_words=fixed_words)
    return results


def _launch_scalar_mul_add_compressed_compressed(data, other, alpha, dense_output):
    device = data.data.device
    _, _, rare_a = get_distribution_tables(data.distribution, device)
    _, _, rare_b = get_distribution_tables(other.distribution, device)
    if rare_a != rare_b:
        raise ValueError("two-compressed path requires matching RARE_LENGTH")
    block_symbols, lanes, steps, fixed_words = data.codec_geometry
    output, auxiliary = _outputs(data, dense_output)
    if data.logical_numel:
        dispatch.dual_scale_add(
            operand_of(data), operand_of(other), output, auxiliary, _scalar(alpha, device),
            data.size, compressed_output=not dense_output, rare_length=rare_a,
            logical_numel=data.logical_numel, block_symbols=block_symbols, lanes=lanes,
            steps=steps, fixed_words=fixed_words,
        )
    return output, auxiliary


def pointwise_scale_add_compressed(
    data: CompressedTensor, other: CompressedTensor, alpha: Tensor, *,
    dense_output: bool = True, buffer: TensorBuffer | None = None,
    distribution: Distribution | None = None,
) -> Tensor | CompressedTensor:
    """``alpha * compA + compB``, dense BF16 or compressed result."""
    both_compressed = (data.layout == StorageLayout.COMPRESSED
                       and other.layout == StorageLayout.COMPRESSED)
    assert (data.fallback_descriptor is None) == (other.fallback_descriptor is None), (
        "pointwise_scale_add_compressed requires both inputs to be buffer-backed "
        "or both to be non-buffer-backed"
    )
    if both_compressed and data.codec_geometry == other.codec_geometry:
        result_distribution = distribution or data.distribution
        if not dense_output and geometry(result_distribution) != data.codec_geometry:
            raise ValueError("matrix compressed output must preserve the input stream geometry")
        values, auxiliary = _launch_scalar_mul_add_compressed_compressed(
            data, other, alpha, dense_output)
        if dense_output:
            return values.reshape(data.shape)
        return compress_components(
            auxiliary, values, data.size, result_distribution, buffer, data.shape,
            precomputed=True, logical_numel=data.logical_numel,
        )
    other_dense = (other.data.reshape(other.shape) if other.layout == StorageLayout.RAW
                   else decode_dense(other))
    return pointwise_compressed_dense(
        data, other_dense, SCALAR_MUL_ADD, alpha=alpha, dense_output=dense_output,
        buffer=buffer, distribution=distribution,
    )


def _raw_result(data, other, operation, alpha, beta, alpha_is_one):
    """Same arithmetic on an uncompressed (RAW layout) left operand, in PyTorch."""
    left = data.data.reshape(data.shape)
    if operation.name != "scalar_mul_add":
        return operation.torch_fn(left, other)
    if alpha_is_one:
        if beta is None:
            return (left.float() + other.float()).to(torch.bfloat16)
        return torch.addcmul(left.float(), other.float(), beta).to(torch.bfloat16)
    if beta is None:
        return operation.torch_fn(left, other, alpha)
    return torch.addcmul(other.float() * beta, left.float(), alpha).to(torch.bfloat16)


def pointwise_compressed_dense(
    data: CompressedTensor, other: Tensor, operation: PointwiseOp, *,
    alpha: Tensor | None = None, beta: Tensor | None = None, alpha_is_one: bool = False,
    dense_output: bool = True, buffer: TensorBuffer | None = None,
    distribution: Distribution | None = None,
) -> Tensor | CompressedTensor:
    """``compA + B``, ``compA * B`` or ``alpha * compA + beta * B`` elementwise."""
    if tuple(other.shape) != data.shape:
        raise ValueError(f"{operation.name} expects tensors with the same shape")
    result_distribution = distribution or data.distribution
    if operation.name == "scalar_mul_add" and alpha is None:
        raise ValueError("scalar_mul_add requires an alpha argument")
    if (data.layout == StorageLayout.COMPRESSED and not dense_output
            and geometry(result_distribution) != data.codec_geometry):
        raise ValueError("matrix compressed output must preserve the input stream geometry")

    if data.layout == StorageLayout.RAW:
        result = _raw_result(data, other, operation, alpha, beta, alpha_is_one)
        return result if dense_output else compress_dense(result, result_distribution, buffer)

    if not dense_output and FUSED_UPDATE and data.logical_numel:
        return _fused_update(data, other, operation, result_distribution, buffer, alpha=alpha,
                             beta=beta, alpha_is_one=alpha_is_one)
    values, auxiliary = _launch_pointwise_compressed_dense(
        data, other, operation, dense_output, alpha=alpha, beta=beta, alpha_is_one=alpha_is_one)
    if dense_output:
        return values.reshape(data.shape)
    return compress_components(
        auxiliary, values, data.size, result_distribution, buffer, data.shape,
        precomputed=True, logical_numel=data.logical_numel,
    )
