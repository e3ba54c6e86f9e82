"""One Python wrapper per launch of the CUDA library.

The function names and argument meaning follow the reference's launch layer
(``LCT/kernels/dispatch.py:16-361``), which is what its host pipelines call;
here each wrapper forwards raw device pointers, sizes and the current CUDA
stream to the C ABI declared in ``include/lct_b200.h``.  Differences from the
reference's layer, all invisible to the pipelines' results:

* overflow rows of the fused operations are handled inside ``pointwise_dense``
  and ``dual_scale_add`` (no separate fix-up launch, no per-stream maps);
* the decoders use two-symbol lookup tables per codebook (one per possible
  center), cached per device by ``pair_table_for``;
* ``compress_pipeline`` and ``update_pipeline`` put all launches of a buffered
  compression / fused update behind one call;
* every launch goes to ``torch.cuda.current_stream`` of the tensors' device.
"""
from __future__ import annotations

import ctypes

import torch

from .. import config
from ..compression.huffman_tables import FIRST_BITS, get_distribution_tables
from . import _lib
from ._lib import DecodeJob, EncodeJob, Operand, Overflow, UpdateJob
from .backends import FallbackStorage

OP_ADD, OP_MULTIPLY, OP_SCALAR_MUL_ADD, OP_LERP, OP_EMA_SQUARE = 0, 1, 2, 3, 4
EMIT_NONE, EMIT_RESULT, EMIT_NESTEROV = 0, 1, 2


def _ptr(tensor: torch.Tensor | None) -> int | None:
    if tensor is None or tensor.numel() == 0:
        return None
    return tensor.data_ptr()


def _require_cuda(tensor: torch.Tensor) -> torch.device:
    if tensor.device.type != "cuda":
        raise ValueError(f"LCT kernel dispatch requires a CUDA device, got {tensor.device}")
    config.check()
    return tensor.device


class _on:
    """Make ``device`` current for a launch when it is not already."""

    def __init__(self, device: torch.device):
        self.guard = None
        if device.index is not None and device.index != torch.cuda.current_device():
            self.guard = torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


try:  # raw handle of the current stream without building a torch.cuda.Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover - older/newer torch without the private helper
    def _raw_stream(index: int) -> int:
        return torch.cuda.current_stream(index).cuda_stream

_functions: dict = {}
_applied_lane_mapping = "swizzle"   # what the library was last told (its own default)


def _apply_lane_mapping() -> None:
    """Hand ``config.lane_mapping`` to the library when it changed since the last launch."""
    global _applied_lane_mapping
    config.check()
    _lib.check(_lib.load().lct_set_lane_mapping(1 if config.lane_mapping == "linear" else 0),
               "lct_set_lane_mapping")
    _applied_lane_mapping = config.lane_mapping


def _call(name: str, device: torch.device, *args, launches: int = 1) -> None:
    """Launch entry point ``name`` (``launches`` kernels) on the current stream of ``device``."""
    function = _functions.get(name)
    if function is None:
        function = _functions[name] = getattr(_lib.load(), name)
    if config.lane_mapping != _applied_lane_mapping:
        _apply_lane_mapping()
    index = device.index
    if index is None:
        index = torch.cuda.current_device()
    if index == torch.cuda.current_device():
        code = function(*args, _raw_stream(index))
        if code:
            _lib.check(code, name)
        return
    with _on(device):
        _lib.check(function(*args, torch.cuda.current_stream(device).cuda_stream), name)


# ---------------------------------------------------------------------------
# Table preparation
# ---------------------------------------------------------------------------

_pair_tables: dict = {}


def pair_table_for(distribution, device: torch.device) -> torch.Tensor:
    """Two-symbol decode tables of a codebook on ``device``: one 4096-entry table per possible
    center, uint32[256 * 4096] stored as int32 (4 MiB, built once)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (distribution.family, distribution.param, distribution.mean, distribution.zero_prob, device)
    table = _pair_tables.get(key)
    if table is None:
        _, decode_table, rare_length = get_distribution_tables(distribution, device)
        table = torch.empty(256 * 4096, dtype=torch.int32, device=device)
        _call(
            "lct_build_pair_table", device,
            decode_table.data_ptr(), rare_length, table.data_ptr())
        _pair_tables[key] = table
    return table


def shift_encoding_table(encode_table, center, shifted_encode, decode_table, shifted_decode=None):
    """Tables for a known center (device int32 scalar)."""
    device = _require_cuda(encode_table)
    if shifted_decode is None:
        shifted_decode = torch.empty_like(decode_table)
    _call(
        "lct_shift_tables", device,
        encode_table.data_ptr(), decode_table.data_ptr(), center.data_ptr(),
        shifted_encode.data_ptr(), shifted_decode.data_ptr())


def estimate_and_shift_encoding_table(source, center, size, encode_table, shifted_encode,
                                      decode_table, shifted_decode, sample_size, precomputed):
    """Sample the center of ``source`` and build both shifted tables in one launch.

    ``sample_size`` is implied (min(size, 4096)) and only checked.
    """
    device = _require_cuda(source)
    if sample_size != min(size, 4096):
        raise ValueError("the center is always estimated from min(size, 4096) samples")
    if shifted_decode is None:
        shifted_decode = torch.empty_like(decode_table)
    _call(
        "lct_center_and_tables", device,
        _ptr(source), size, int(precomputed), encode_table.data_ptr(), decode_table.data_ptr(),
        center.data_ptr(), shifted_encode.data_ptr(), shifted_decode.data_ptr())


def shift_decoding_table(decode_table, center):
    """Return a center-shifted copy of ``decode_table``."""
    device = _require_cuda(decode_table)
    shifted = torch.empty(1 << FIRST_BITS, dtype=torch.int32, device=device)
    _call(
        "lct_shift_tables", device,
        None, decode_table.data_ptr(), center.data_ptr(), None, shifted.data_ptr())
    return shifted


# ---------------------------------------------------------------------------
# Encode pipeline
# ---------------------------------------------------------------------------

def encode_kernel(source, side, encoded, encode_table, extra_starts, summaries, size, streams, *,
                  precomputed, logical_numel, block_symbols, lanes, steps, fixed_words,
                  write_summary=True):
    """Field split + Huffman encode; always writes the per-block overflow summaries."""
    device = _require_cuda(source)
    if lanes != 256 or streams != size // block_symbols * lanes:
        raise ValueError("inconsistent stream geometry")
    _call(
        "lct_encode", device,
        _ptr(source), _ptr(side), encoded.data_ptr(), encode_table.data_ptr(),
        extra_starts.data_ptr(), summaries.data_ptr(), size, logical_numel, block_symbols,
        steps, fixed_words, int(precomputed))


def prefix_allocate(summaries, counts, descriptor, buffer, blocks, buffered, max_free_regions):
    """Scan the block summaries and, when ``buffered``, reserve the shared arena region."""
    device = _require_cuda(summaries)
    storage = buffer._storage.data_ptr() if buffered else None
    _call(
        "lct_scan_allocate", device,
        summaries.data_ptr(), counts.data_ptr(), descriptor.data_ptr() if buffered else None,
        storage, blocks, max_free_regions)


def compress_pipeline(source, side, encoded, encode_table, decode_table, center, shifted_encode,
                      shifted_decode, extra_starts, summaries, counts, descriptor, blocks_out,
                      buffer, size, *, precomputed, logical_numel, block_symbols, steps,
                      fixed_words):
    """Center, encode, scan + arena reservation and tail compaction of one tensor as one call
    (four launches that overlap where their data allows); same bytes as the four wrappers
    ``estimate_and_shift_encoding_table``, ``encode_kernel``, ``prefix_allocate`` and
    ``compact_extra`` called in that order with a shared ``buffer``."""
    device = _require_cuda(source)
    _call(
        "lct_compress", device,
        _ptr(source), int(precomputed), _ptr(side), encoded.data_ptr(), encode_table.data_ptr(),
        decode_table.data_ptr(), center.data_ptr(), shifted_encode.data_ptr(),
        shifted_decode.data_ptr(), extra_starts.data_ptr(), summaries.data_ptr(),
        counts.data_ptr(), descriptor.data_ptr(), blocks_out.data_ptr(),
        buffer._storage.data_ptr(), buffer.max_free_regions, size, logical_numel, block_symbols,
        steps, fixed_words, launches=4)


def compact_extra(source, storage: FallbackStorage, final_counts, n_blocks, n_elements, *,
                  precomputed, buffered, logical_numel, block_symbols, lanes, steps,
                  extra_starts, summaries, n_streams, build_meta=True):
    """Write overflow entries, raw exponent tails and the per-block metadata."""
    device = _require_cuda(source)
    if not build_meta:
        raise ValueError("only the summaries path (build_meta=True) exists")
    _call(
        "lct_compact_tails", device,
        _ptr(source), _ptr(storage.lanes), _ptr(storage.starts), _ptr(storage.tail),
        storage.descriptor.data_ptr() if buffered else None, final_counts.data_ptr(),
        storage.blocks.data_ptr(), extra_starts.data_ptr(), summaries.data_ptr(),
        n_elements, logical_numel, block_symbols, steps, int(precomputed))


# ---------------------------------------------------------------------------
# Decode and fused operations
# ---------------------------------------------------------------------------

def fallback_tail_args(storage: FallbackStorage | None) -> Overflow:
    """The overflow view the decoders take (``struct lct_overflow``)."""
    view = Overflow()
    if storage is None:
        view.mode = 0
        return view
    view.lanes = _ptr(storage.lanes)
    view.starts = _ptr(storage.starts)
    view.tail = _ptr(storage.tail)
    view.count = _ptr(storage.count)
    view.blocks = _ptr(storage.blocks)
    view.base = int(storage.base)
    if storage.buffered:
        view.descriptor = storage.descriptor.data_ptr()
        view.mode = 2
    else:
        view.mode = 1
    return view


def make_operand(encoded, side, shifted_decode, center, pair_table, overflow: Overflow) -> Operand:
    operand = Operand()
    operand.encoded = encoded.data_ptr()
    operand.side = side.data_ptr()
    operand.shifted_decode = shifted_decode.data_ptr() if shifted_decode is not None else None
    operand.center = center.data_ptr()
    operand.pair_table = pair_table.data_ptr()
    operand.overflow = overflow
    return operand


def decode_kernel(operand: Operand, output, size, *, logical_numel, block_symbols, lanes, steps,
                  fixed_words, rare_length):
    """Decode into ``output`` (int16[logical_numel]); overflow tails restored in the same launch."""
    device = _require_cuda(output)
    _call(
        "lct_decode", device,
        ctypes.byref(operand), output.data_ptr(), size, logical_numel, block_symbols, steps,
        fixed_words, rare_length)


def pointwise_dense(operand: Operand, other, output, auxiliary, n_elements, alpha, beta, *,
                    op, alpha_is_one, beta_is_one, compressed_output, rare_length, logical_numel,
                    block_symbols, lanes, steps, fixed_words):
    """Decode one compressed operand, apply ``op`` against dense ``other``, emit dense BF16
    or (side bytes, exponent bytes) for re-encoding."""
    device = _require_cuda(output)
    _call(
        "lct_pointwise", device,
        ctypes.byref(operand), other.data_ptr(), output.data_ptr(),
        auxiliary.data_ptr() if compressed_output else None,
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        op, int(alpha_is_one), int(beta_is_one), int(compressed_output), n_elements,
        logical_numel, block_symbols, steps, fixed_words, rare_length)


def update_sample(operand: Operand, other, samples, n_elements, alpha, beta, *, op, alpha_is_one,
                  beta_is_one, rare_length, logical_numel, block_symbols, lanes, steps,
                  fixed_words, known_values=None, result_values=None):
    """Exponent bytes of ``compA (op) other`` at the positions the center estimate samples.
    ``result_values`` (int16[samples]) receives the full BF16 results there; ``known_values`` are
    such values of ``compA`` kept from the update that produced it (no stream walk then)."""
    device = _require_cuda(samples)
    _call(
        "lct_update_sample", device,
        ctypes.byref(operand), other.data_ptr(),
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        op, int(alpha_is_one), int(beta_is_one), samples.data_ptr(), _ptr(known_values),
        _ptr(result_values), n_elements, logical_numel, block_symbols, steps, fixed_words,
        rare_length)


def update_fused(operand: Operand, other, shifted_encode, side_out, encoded_out, extra_starts,
                 summaries, spill, n_elements, alpha, beta, *, op, alpha_is_one, beta_is_one,
                 rare_length, logical_numel, block_symbols, lanes, steps, fixed_words):
    """Decode, apply ``op`` against dense ``other`` and re-encode in one launch."""
    device = _require_cuda(side_out)
    _call(
        "lct_update_fused", device,
        ctypes.byref(operand), other.data_ptr(),
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        op, int(alpha_is_one), int(beta_is_one), shifted_encode.data_ptr(), side_out.data_ptr(),
        encoded_out.data_ptr(), extra_starts.data_ptr(), summaries.data_ptr(), spill.data_ptr(),
        n_elements, logical_numel, block_symbols, steps, fixed_words, rare_length)


def update_pipeline(operand: Operand, other, alpha, beta, encode_table, decode_table, samples,
                    center, shifted_encode, shifted_decode, side_out, encoded_out, extra_starts,
                    summaries, spill, counts, descriptor, blocks_out, buffer, n_elements, *, op,
                    alpha_is_one, beta_is_one, rare_length, logical_numel, block_symbols, lanes,
                    steps, fixed_words, known_values=None, result_values=None):
    """Sample, center, decode-op-encode, scan + reservation and tail compaction of a fused update
    as one call (five launches that overlap where their data allows)."""
    device = _require_cuda(side_out)
    _call(
        "lct_update", device,
        ctypes.byref(operand), other.data_ptr(),
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        op, int(alpha_is_one), int(beta_is_one), encode_table.data_ptr(), decode_table.data_ptr(),
        samples.data_ptr(), _ptr(known_values), _ptr(result_values), center.data_ptr(),
        shifted_encode.data_ptr(), shifted_decode.data_ptr(), side_out.data_ptr(),
        encoded_out.data_ptr(),
        extra_starts.data_ptr(), summaries.data_ptr(), spill.data_ptr(), counts.data_ptr(),
        descriptor.data_ptr(), blocks_out.data_ptr(), buffer._storage.data_ptr(),
        buffer.max_free_regions, n_elements, logical_numel, block_symbols, steps, fixed_words,
        rare_length, launches=5)


def dual_scale_add(a: Operand, b: Operand, output, auxiliary, alpha, n_elements, *,
                   compressed_output, rare_length, logical_numel, block_symbols, lanes, steps,
                   fixed_words):
    """``alpha * compA + compB`` in one launch."""
    device = _require_cuda(output)
    _call(
        "lct_dual_scale_add", device,
        ctypes.byref(a), ctypes.byref(b), output.data_ptr(),
        auxiliary.data_ptr() if compressed_output else None, alpha.data_ptr(),
        int(compressed_output), n_elements, logical_numel, block_symbols, steps, fixed_words,
        rare_length)


# ---------------------------------------------------------------------------
# Many tensors per launch
# ---------------------------------------------------------------------------

def _to_device(records, device: torch.device) -> torch.Tensor:
    """A ctypes array of job records as a device byte tensor.  Staged through pinned memory so
    that the copy is asynchronous: from pageable memory the host would wait for everything
    queued on the stream before it could go on preparing the next call."""
    nbytes = ctypes.sizeof(records)
    staged = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    ctypes.memmove(staged.data_ptr(), ctypes.addressof(records), nbytes)
    return staged.to(device, non_blocking=True)


class CompressBatch:
    """A prepared multi-tensor compression: the device job table and work buffers.  ``run`` may
    be called any number of times (e.g. once per training step) as long as the tensors the jobs
    point at stay alive and in place."""

    def __init__(self, jobs: list[dict], encode_table, decode_table, buffer, *, block_symbols,
                 lanes, steps, fixed_words):
        self.device = _require_cuda(encode_table)
        records = (EncodeJob * len(jobs))()
        first = 0
        for record, job in zip(records, jobs):
            record.src = job["src"].data_ptr()
            record.side = job["side"].data_ptr()
            record.encoded = job["encoded"].data_ptr()
            record.center = job["center"].data_ptr()
            record.shifted_decode = job["decode_table"].data_ptr()
            record.counts = job["counts"].data_ptr()
            record.descriptor = job["descriptor"].data_ptr()
            record.blocks_out = job["blocks"].data_ptr()
            record.size = job["size"]
            record.logical_numel = job["logical_numel"]
            record.first_block = first
            first += job["size"] // block_symbols
        self.keep = (jobs, encode_table, decode_table, buffer)
        self.table = _to_device(records, self.device)
        self.extra_starts = torch.empty(first * lanes, dtype=torch.uint8, device=self.device)
        self.summaries = torch.empty(4 * first, dtype=torch.int32, device=self.device)
        self.shifted_encode = torch.empty(256 * len(jobs), dtype=torch.int32, device=self.device)
        self.args = (
            self.table.data_ptr(), len(jobs), first, encode_table.data_ptr(),
            decode_table.data_ptr(), buffer._storage.data_ptr(), buffer.max_free_regions,
            self.extra_starts.data_ptr(), self.summaries.data_ptr(),
            self.shifted_encode.data_ptr(), block_symbols, steps, fixed_words)

    def run(self) -> None:
        _call("lct_compress_batch", self.device, *self.args, launches=4)


def compress_batch(jobs: list[dict], encode_table, decode_table, buffer, **geometry_kw):
    """Compress many tensors of one codebook and geometry into ``buffer``'s arena with four
    launches.  Each job is a dict of tensors: ``src`` (int16 bits, contiguous), ``side``,
    ``encoded``, ``center``, ``decode_table``, ``counts``, ``descriptor``, ``blocks`` plus
    ``size`` and ``logical_numel``.  Returns the prepared batch (re-runnable)."""
    batch = CompressBatch(jobs, encode_table, decode_table, buffer, **geometry_kw)
    batch.run()
    return batch


def update_batch(jobs: list[dict], alpha, beta, encode_table, decode_table, buffer, *, op,
                 alpha_is_one, beta_is_one, rare_length, block_symbols, lanes, steps, fixed_words):
    """Fused update of many compressed tensors of one codebook and geometry into ``buffer``'s
    arena with five launches in all (instead of five per tensor).  Each job is a dict: ``operand``
    (the state), ``other`` (dense BF16), ``known_values`` / ``result_values`` (or None),
    ``side_out``, ``encoded_out``, ``spill``, ``center``, ``decode_table``, ``counts``,
    ``descriptor``, ``blocks`` plus ``size`` and ``logical_numel``.  Returns the work tensors,
    which must stay referenced until the launches have run."""
    device = _require_cuda(encode_table)
    records = (UpdateJob * len(jobs))()
    first = 0
    for record, job in zip(records, jobs):
        record.a = job["operand"]
        record.other = job["other"].data_ptr()
        record.known_values = _ptr(job.get("known_values"))
        record.result_values = _ptr(job.get("result_values"))
        record.side_out = job["side_out"].data_ptr()
        record.encoded_out = job["encoded_out"].data_ptr()
        record.spill = job["spill"].data_ptr()
        record.center = job["center"].data_ptr()
        record.shifted_decode = job["decode_table"].data_ptr()
        record.counts = job["counts"].data_ptr()
        record.descriptor = job["descriptor"].data_ptr()
        record.blocks_out = job["blocks"].data_ptr()
        record.size = job["size"]
        record.logical_numel = job["logical_numel"]
        record.first_block = first
        first += job["size"] // block_symbols
    table = _to_device(records, device)
    work = torch.empty(4096 * len(jobs) + first * lanes + 16, dtype=torch.uint8, device=device)
    samples, extra_starts = work[:4096 * len(jobs)], work[4096 * len(jobs):]
    ints = torch.empty(4 * first + 256 * len(jobs), dtype=torch.int32, device=device)
    summaries, shifted_encode = ints[:4 * first], ints[4 * first:]
    _call(
        "lct_update_batch", device,
        table.data_ptr(), len(jobs), first,
        alpha.data_ptr() if alpha is not None else None,
        beta.data_ptr() if beta is not None else None,
        op, int(alpha_is_one), int(beta_is_one), encode_table.data_ptr(), decode_table.data_ptr(),
        buffer._storage.data_ptr(), buffer.max_free_regions, samples.data_ptr(),
        shifted_encode.data_ptr(), extra_starts.data_ptr(), summaries.data_ptr(), block_symbols,
        steps, fixed_words, rare_length, launches=5)
    return table, work, ints


class DecodeBatch:
    """A prepared multi-tensor decode (one launch per ``run``).  Each job is
    ``(operand, output int16 tensor, size, logical_numel)`` with an optional fifth element: a
    local uint8 tensor of ``size`` bytes through which the job's side bytes are staged (for
    operands in a peer GPU's memory)."""

    def __init__(self, jobs: list[tuple], *, block_symbols, lanes, steps, fixed_words, rare_length):
        self.device = _require_cuda(jobs[0][1])
        records = (DecodeJob * len(jobs))()
        first = 0
        for record, job in zip(records, jobs):
            operand, output, size, logical_numel = job[:4]
            stage = job[4] if len(job) > 4 else None
            if output.data_ptr() % 16:
                raise ValueError("batched decode needs 16-byte aligned outputs")
            if stage is not None:
                if stage.numel() < size or stage.data_ptr() % 16 or stage.device != output.device:
                    raise ValueError("side-byte stage must be a local, 16-byte aligned tensor of "
                                     "at least `size` bytes")
                record.side_stage = stage.data_ptr()
            record.operand = operand
            record.out = output.data_ptr()
            record.size = size
            record.logical_numel = logical_numel
            record.first_block = first
            first += size // block_symbols
        self.keep = jobs
        self.table = _to_device(records, self.device)
        self.args = (self.table.data_ptr(), len(jobs), first, block_symbols, steps, fixed_words,
                     rare_length)

    def run(self) -> None:
        _call("lct_decode_batch", self.device, *self.args)


def decode_batch(jobs: list[tuple], **geometry_kw):
    """Decode many compressed tensors of one geometry in one launch."""
    batch = DecodeBatch(jobs, **geometry_kw)
    batch.run()
    return batch


# ---------------------------------------------------------------------------
# Shared arena
# ---------------------------------------------------------------------------

def buffer_reset(storage, max_free_regions, capacity_bytes):
    device = _require_cuda(storage)
    _call(
        "lct_buffer_reset", device,
        storage.data_ptr(), max_free_regions, capacity_bytes)


def buffer_allocate(storage, requested_bytes, item_count, item_bytes, descriptor, max_free_regions):
    device = _require_cuda(storage)
    _call(
        "lct_buffer_allocate", device,
        storage.data_ptr(), requested_bytes.data_ptr(),
        item_count.data_ptr() if item_count is not None else None, item_bytes,
        descriptor.data_ptr(), max_free_regions)


def buffer_free(storage, descriptor, status, max_free_regions):
    device = _require_cuda(storage)
    _call(
        "lct_buffer_free", device,
        storage.data_ptr(), descriptor.data_ptr(), status.data_ptr(), max_free_regions)
