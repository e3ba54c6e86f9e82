"""A prepared in-place update of a fixed list of compressed tensors.

``LCTTensor.mul_add_`` (reference: ``LCT/LCTensor.py:79-95``) builds a new compressed value per
call: about a dozen small allocations, an operand record and five launches per tensor, which is
more host time than the GPU needs for a 16 Mi-element tensor.  An optimizer applies the same
update to the same tensors every step, so everything but the launches can be prepared once:

    plan = UpdatePlan(momentums, alpha)          # list of LCTTensor sharing one arena
    plan.step(grads)                             # m_i <- alpha * m_i + g_i, every step

The same for the other fused operations: ``UpdatePlan(momentums, one_minus_mu, mu,
operation=LERP, emit=EMIT_NESTEROV)`` with ``plan.step(grads, dense_outs=grads)`` is the momentum
step of every parameter of Muon in one call, the Nesterov directions overwriting the gradients
(``LCT/components/sparse_utils.py:88-90``).

The plan owns two sets of result storage per tensor that alternate (step k reads one and writes
the other), the device job tables of ``lct_update_batch`` for both directions and the work
buffers.  A step is one call of five launches for the whole list plus one launch that returns the
old values' arena regions.  The values, the compressed bytes and the arena reservations are those
of ``LCTTensor.mul_add_many_(..., group=None)``.

What a caller must know: after ``step`` each ``tensor.x`` is one of the plan's two values for that
tensor, and the value it held before is overwritten by the step after next - keep no reference to
an old ``tensor.x`` across two steps.  Between steps the tensors may be read (``decompress``) but
not replaced; a tensor whose ``x`` was changed behind the plan's back makes ``step`` raise.
"""
from __future__ import annotations

import torch

from .codec import pointwise as _pointwise
from .codec.decode import operand_of
from .codec.geometry import geometry
from .comp_format import StorageLayout
from .comp_tensor import CompressedTensor
from .compression.huffman_tables import get_distribution_tables
from .kernels import dispatch
from .kernels._lib import UpdateJob


class UpdatePlan:
    def __init__(self, tensors, alpha, beta=None, *, alpha_is_one: bool = False,
                 operation=None, emit: int = dispatch.EMIT_NONE, distribution=None):
        """``operation``: ``pointwise.SCALAR_MUL_ADD`` (default), ``LERP`` (``alpha`` = weight) or
        ``EMA_SQUARE``.  ``emit``: every step also writes a dense BF16 by-product per tensor (the
        new value, or with ``LERP`` the Nesterov direction ``lerp(update, new value, beta)``) to
        the ``dense_outs`` given to ``step``.  ``distribution``: the codebook of the results when
        it is not the tensors' own (same stream geometry), e.g. a momentum that was first
        compressed with the many-zeros codebook."""
        self.tensors = list(tensors)
        if not self.tensors:
            raise ValueError("UpdatePlan needs at least one tensor")
        first = self.tensors[0].x
        self.buffer = first.buffer
        if self.buffer is None or self.buffer.capacity_bytes % 4:
            raise ValueError("UpdatePlan needs tensors compressed into a TensorBuffer whose "
                             "capacity is divisible by 4")
        self.device = first.data.device
        self.distribution = distribution or first.distribution
        self.geometry = first.codec_geometry
        if geometry(self.distribution) != self.geometry:
            raise ValueError("the results' codebook must have the tensors' stream geometry")
        for tensor in self.tensors:
            x = tensor.x
            if (x.layout != StorageLayout.COMPRESSED or x.distribution != first.distribution
                    or x.codec_geometry != self.geometry or x.data.device != self.device
                    or x.buffer is not self.buffer or not x.logical_numel):
                raise ValueError("UpdatePlan needs non-empty compressed tensors of one codebook, "
                                 "geometry, device and arena")
        self.operation = operation or _pointwise.SCALAR_MUL_ADD
        scaled = self.operation is _pointwise.SCALAR_MUL_ADD
        if not scaled and alpha_is_one:
            raise ValueError("alpha_is_one belongs to scalar_mul_add")
        if self.operation is _pointwise.EMA_SQUARE and beta is None:
            raise ValueError("ema_square requires a beta argument")
        if emit == dispatch.EMIT_NESTEROV and (self.operation is not _pointwise.LERP or beta is None):
            raise ValueError("the Nesterov direction needs the lerp operation and its weight (beta)")
        self.emit = emit
        self.alpha = None if alpha_is_one else _pointwise._scalar(alpha, self.device)
        self.beta = None if beta is None else _pointwise._scalar(beta, self.device)
        self.alpha_is_one = alpha_is_one
        self.encode_table, self.decode_table, _ = get_distribution_tables(
            self.distribution, self.device)
        block_symbols, lanes, _, _ = self.geometry
        self.sizes = [t.x.size for t in self.tensors]
        self.total_blocks = sum(self.sizes) // block_symbols
        n = len(self.tensors)

        def new(count, dtype):
            return torch.empty(count, dtype=dtype, device=self.device)

        self.values = [[self._new_value(t.x, new) for t in self.tensors] for _ in range(2)]
        self.spill = new(sum(self.sizes), torch.uint8)           # work buffers, reused every step
        self.samples = new(4096 * n, torch.uint8)
        self.extra_starts = new(self.total_blocks * lanes, torch.uint8)
        self.summaries = new(4 * self.total_blocks, torch.int32)
        self.shifted_encode = new(256 * n, torch.int32)
        self.status = new(n, torch.int32)
        # device arrays of the descriptor pointers of each set, for the one-launch free
        self.descriptor_lists = [
            torch.tensor([v.fallback_descriptor.data_ptr() for v in values], dtype=torch.int64)
            .to(self.device) for values in self.values]
        self.which = 0            # the set the next step writes
        self.tables: dict = {}    # (source set, target set) -> [records, device table, others]

    def _new_value(self, like: CompressedTensor, new) -> CompressedTensor:
        block_symbols, lanes, _, fixed_words = self.geometry
        blocks = like.size // block_symbols
        counts = new(4, torch.int32)
        value = CompressedTensor(
            new(blocks * lanes * fixed_words + 4, torch.int32), like.size,
            new(like.size, torch.uint8), fallback_starts=None, fallback_lanes=None,
            fallback_blocks=new(3 * blocks, torch.int32), fallback_buffer=self.buffer.data,
            fallback_descriptor=new(4, torch.int32), buffer=self.buffer,
            fallback_count=counts[:1], fallback_used=counts[1:2], distribution=self.distribution,
            center=new(1, torch.int32), decode_table=new(self.decode_table.numel(), torch.int32),
            shape=like.shape, layout=StorageLayout.COMPRESSED,
            stream_geometry=geometry(self.distribution))
        object.__setattr__(value, _pointwise._SAMPLE_VALUES,
                           new(min(like.logical_numel, 4096), torch.int16))
        object.__setattr__(value, "_b200_counts", counts)
        return value

    def _table(self, sources, source_key, others, dense_outs):
        """Job table for ``sources -> self.values[self.which]`` with the dense operands at
        ``others`` and the by-products at ``dense_outs`` (pointers); rebuilt only when a pointer
        in it changed."""
        key = (source_key, self.which)
        entry = self.tables.get(key)
        if entry is not None and entry[2] == (others, dense_outs):
            return entry[1]
        block_symbols = self.geometry[0]
        records = (UpdateJob * len(sources))()
        first = at = 0
        for record, source, target, other, dense_out in zip(records, sources,
                                                            self.values[self.which], others,
                                                            dense_outs):
            known = getattr(source, _pointwise._SAMPLE_VALUES, None)
            count = min(source.logical_numel, 4096)
            if known is not None and (known.numel() != count or known.device != self.device):
                known = None
            record.a = operand_of(source)
            record.other = other
            record.known_values = known.data_ptr() if known is not None else None
            record.result_values = getattr(target, _pointwise._SAMPLE_VALUES).data_ptr()
            record.side_out = target.sign_mantissa.data_ptr()
            record.encoded_out = target.data.data_ptr()
            record.spill = self.spill.data_ptr() + at
            record.center = target.center.data_ptr()
            record.shifted_decode = target.decode_table.data_ptr()
            record.counts = getattr(target, "_b200_counts").data_ptr()
            record.descriptor = target.fallback_descriptor.data_ptr()
            record.blocks_out = target.fallback_blocks.data_ptr()
            record.size = source.size
            record.logical_numel = source.logical_numel
            record.first_block = first
            record.dense_out = dense_out
            first += source.size // block_symbols
            at += source.size
        table = dispatch._to_device(records, self.device)
        if source_key != "own":
            # Values of the plan never move, so the table stays good while the updates do.  A
            # table that reads the tensors' own first values is built for that one step only.
            self.tables[key] = [records, table, (others, dense_outs)]
        return table

    def step(self, updates, dense_outs=None) -> None:
        """``x_i <- x_i (op) updates[i]`` for every tensor of the plan (default operation:
        ``alpha * x_i + beta * updates[i]``); with ``emit`` the by-product of tensor i goes to
        ``dense_outs[i]`` (contiguous BF16 of the tensor's shape; may be ``updates[i]`` itself)."""
        if len(updates) != len(self.tensors):
            raise ValueError("UpdatePlan.step needs one update per tensor")
        if self.emit != dispatch.EMIT_NONE:
            if dense_outs is None or len(dense_outs) != len(self.tensors):
                raise ValueError("this plan writes a dense by-product per tensor: pass dense_outs")
            for tensor, out in zip(self.tensors, dense_outs):
                if (out.dtype != torch.bfloat16 or out.device != self.device
                        or tuple(out.shape) != tensor.x.shape or not out.is_contiguous()
                        or out.data_ptr() % 16):
                    raise ValueError("dense_outs must be contiguous, 16-byte aligned bfloat16 "
                                     "tensors of the tensors' shapes on their device")
            out_pointers = [out.data_ptr() for out in dense_outs]
        else:
            out_pointers = [None] * len(self.tensors)
        sources = [tensor.x for tensor in self.tensors]
        previous = self.values[1 - self.which]
        if all(s is p for s, p in zip(sources, previous)):
            source_key = 1 - self.which
        elif any(s is v for s in sources for values in self.values for v in values):
            raise ValueError("a tensor of the plan was changed between steps")
        else:
            source_key = "own"    # first step, or the caller re-compressed every tensor
            if any(s.distribution != sources[0].distribution or s.codec_geometry != self.geometry
                   or s.buffer is not self.buffer for s in sources):
                raise ValueError("UpdatePlan needs tensors of one codebook, geometry and arena")
        flat = []
        for source, update in zip(sources, updates):
            if tuple(update.shape) != source.shape:
                raise ValueError("scalar_mul_add expects tensors with the same shape")
            if update.dtype != torch.bfloat16:
                raise TypeError("the dense operand must be bfloat16")
            flat.append(update.contiguous())
        table = self._table(sources, source_key, [u.data_ptr() for u in flat], out_pointers)
        block_symbols, lanes, steps, fixed_words = self.geometry
        # the escape-prefix length the decoder needs is the SOURCES' codebook's
        _, _, rare_length = get_distribution_tables(sources[0].distribution, self.device)
        scaled = self.operation is _pointwise.SCALAR_MUL_ADD
        dispatch._call(
            "lct_update_batch_emit", self.device,
            table.data_ptr(), len(sources), self.total_blocks,
            self.alpha.data_ptr() if self.alpha is not None else None,
            self.beta.data_ptr() if self.beta is not None else None,
            self.operation.code, int(not scaled or self.alpha_is_one),
            int(not scaled or self.beta is None),
            self.encode_table.data_ptr(), self.decode_table.data_ptr(),
            self.buffer._storage.data_ptr(), self.buffer.max_free_regions,
            self.samples.data_ptr(), self.shifted_encode.data_ptr(), self.extra_starts.data_ptr(),
            self.summaries.data_ptr(), block_symbols, steps, fixed_words, rare_length, self.emit,
            launches=5)
        for tensor, value in zip(self.tensors, self.values[self.which]):
            tensor.x = value
        if source_key == "own":
            for source in sources:
                source.free()
        else:
            dispatch._call(
                "lct_buffer_free_many", self.device,
                self.buffer._storage.data_ptr(), self.descriptor_lists[source_key].data_ptr(),
                len(sources), self.status.data_ptr(), self.buffer.max_free_regions)
        self.which ^= 1
