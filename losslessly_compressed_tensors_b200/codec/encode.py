"""Host pipeline that turns BF16 values (or already split components) into a ``CompressedTensor``.

Launch order and every output allocation follow the reference's
``LCT/codec/encode.py:22-218`` so that the result holds the same tensors with
the same sizes:

1. center sample + shifted tables                       (1 CTA)
2. field split + fixed-budget Huffman encode            (1 CTA per block)
3. scan of per-block overflow summaries (+ arena reservation when buffered)
4. compact overflow entries and raw exponent tails      (1 CTA per block)

With a shared ``TensorBuffer`` nothing synchronises the host.  Without one the
overflow tensors are allocated at their exact size, which needs the two totals
on the host (one 8-byte copy), exactly like the reference.
"""
from __future__ import annotations

import torch

from ..comp_format import Distribution, StorageLayout
from ..comp_tensor import CompressedTensor
from ..compression.huffman_tables import get_distribution_tables
from ..kernels import dispatch
from ..kernels.backends import FallbackStorage
from ..tensor_buffer import TensorBuffer
from .geometry import geometry

CENTER_SAMPLE_SIZE = 4096

# Compress into a shared buffer through the single-call pipeline (``lct_compress``) instead of
# one call per stage.  Same launches, same bytes; the switch exists so that the stages can be
# timed one by one.
SINGLE_CALL_PIPELINE = True


def encode_components(
    source_values: torch.Tensor,
    sign_mantissa: torch.Tensor,
    size: int,
    distribution: Distribution,
    buffer: TensorBuffer | None,
    shape: tuple[int, ...],
    *,
    precomputed: bool,
    center: torch.Tensor | None = None,
    logical_numel: int,
    out=None,
    center_samples: torch.Tensor | None = None,
    launch_encode=None,
) -> CompressedTensor:
    """Encode int16 BF16 bits, or (``precomputed``) uint8 exponent bytes in logical order
    whose side bytes already sit in ``sign_mantissa``.  ``size`` is the padded element count.

    ``out`` (not in the reference): an object with ``take(name, numel, dtype) -> Tensor`` that
    supplies the storage of the buffered result's persistent tensors (``encoded``, ``counts``,
    ``blocks``, ``center``, ``decode_table``, ``descriptor``), e.g. slices of a wire buffer."""
    if buffer is not None and buffer.capacity_bytes % 4:
        raise ValueError("TensorBuffer capacity must be divisible by 4")
    device = source_values.device
    stream_geometry = geometry(distribution)
    block_symbols, lanes, steps, fixed_words = stream_geometry
    blocks = -(-size // block_symbols)
    streams = blocks * lanes
    encode_table, decode_table, _ = get_distribution_tables(distribution, device)

    def scratch(n, dtype):
        return torch.empty(n, dtype=dtype, device=device)

    def kept(name, n, dtype):
        return scratch(n, dtype) if out is None else out.take(name, n, dtype)

    if out is not None and buffer is None:
        raise ValueError("placing the result needs a shared buffer (sizes must not depend on the data)")
    shifted_encode = scratch(256, torch.int32)
    shifted_decode = kept("decode_table", decode_table.numel(), torch.int32)
    if (SINGLE_CALL_PIPELINE and buffer is not None and center is None and center_samples is None
            and launch_encode is None and blocks > 0):
        center = kept("center", 1, torch.int32)
        encoded = kept("encoded", streams * fixed_words + 4, torch.int32)
        extra_starts = scratch(streams, torch.uint8)
        summaries = scratch(4 * blocks, torch.int32)
        counts = kept("counts", 4, torch.int32)
        blocks_out = kept("blocks", 3 * blocks, torch.int32)
        descriptor = kept("descriptor", 4, torch.int32)
        dispatch.compress_pipeline(
            source_values, None if precomputed else sign_mantissa, encoded, encode_table,
            decode_table, center, shifted_encode, shifted_decode, extra_starts, summaries, counts,
            descriptor, blocks_out, buffer, size, precomputed=precomputed,
            logical_numel=logical_numel, block_symbols=block_symbols, steps=steps,
            fixed_words=fixed_words)
        return CompressedTensor(
            encoded, size, sign_mantissa,
            fallback_starts=None, fallback_lanes=None, fallback_blocks=blocks_out,
            fallback_buffer=buffer.data, fallback_descriptor=descriptor, buffer=buffer,
            fallback_count=counts[:1], fallback_used=counts[1:2],
            distribution=distribution, center=center, decode_table=shifted_decode, shape=shape,
            layout=StorageLayout.COMPRESSED, stream_geometry=stream_geometry,
        )
    if center is None:
        center = kept("center", 1, torch.int32)
        if center_samples is None:
            dispatch.estimate_and_shift_encoding_table(
                source_values, center, logical_numel, encode_table, shifted_encode,
                decode_table, shifted_decode, min(logical_numel, CENTER_SAMPLE_SIZE), precomputed,
            )
        else:
            # One sample per position: the estimator then reads every given byte exactly once.
            count = center_samples.numel()
            dispatch.estimate_and_shift_encoding_table(
                center_samples, center, count, encode_table, shifted_encode,
                decode_table, shifted_decode, min(count, CENTER_SAMPLE_SIZE), True,
            )
    else:
        dispatch.shift_encoding_table(encode_table, center, shifted_encode, decode_table,
                                      shifted_decode)

    encoded = kept("encoded", streams * fixed_words + 4, torch.int32)
    extra_starts = scratch(streams, torch.uint8)
    summaries = scratch(4 * blocks, torch.int32)
    counts = kept("counts", 4, torch.int32)
    blocks_out = kept("blocks", 3 * blocks, torch.int32)
    if blocks == 0:
        # Nothing to encode: an empty tensor keeps well-defined (zero) metadata.
        encoded.zero_()
        counts.zero_()
    elif launch_encode is not None:
        launch_encode(shifted_encode, encoded, extra_starts, summaries)
    else:
        dispatch.encode_kernel(
            source_values, sign_mantissa, encoded, shifted_encode, extra_starts, summaries,
            size, streams, precomputed=precomputed, logical_numel=logical_numel,
            block_symbols=block_symbols, lanes=lanes, steps=steps, fixed_words=fixed_words,
        )
    final_count, final_total = counts[:1], counts[1:2]

    buffered = buffer is not None
    if buffered:
        descriptor = kept("descriptor", 4, torch.int32)
        if blocks:
            dispatch.prefix_allocate(summaries, counts, descriptor, buffer, blocks, True,
                                     buffer.max_free_regions)
        else:
            descriptor.copy_(torch.tensor([-1, 0, 2, 0], dtype=torch.int32))
        arena = buffer.data
        storage = FallbackStorage(tail=arena, count=final_count, lanes=arena, starts=arena,
                                  blocks=blocks_out, descriptor=descriptor, allocation=descriptor)
    else:
        descriptor = None
        if blocks:
            dispatch.prefix_allocate(summaries, counts, counts, None, blocks, False, 256)
        # Exact-size private overflow tensors need the two totals on the host.
        count, tail_bytes = (int(v) for v in counts[:2].tolist())
        storage = FallbackStorage(
            tail=scratch(tail_bytes, torch.uint8), count=final_count,
            lanes=scratch(count, torch.uint8), starts=scratch(count, torch.uint8),
            blocks=blocks_out, allocation=counts[2:3], base=0,
        )
    if blocks:
        dispatch.compact_extra(
            source_values, storage, final_count, blocks, size,
            precomputed=precomputed, buffered=buffered, logical_numel=logical_numel,
            block_symbols=block_symbols, lanes=lanes, steps=steps,
            extra_starts=extra_starts, summaries=summaries, n_streams=streams,
        )
    return CompressedTensor(
        encoded, size, sign_mantissa,
        fallback_starts=None if buffered else storage.starts,
        fallback_lanes=None if buffered else storage.lanes,
        fallback_blocks=storage.blocks,
        fallback_buffer=storage.tail,
        fallback_descriptor=descriptor,
        buffer=buffer,
        fallback_count=final_count,
        fallback_used=final_total,
        distribution=distribution, center=center, decode_table=shifted_decode,
        shape=shape,
        layout=StorageLayout.COMPRESSED,
        stream_geometry=stream_geometry,
    )


def encode(data: torch.Tensor, distribution: Distribution, buffer: TensorBuffer | None = None, *,
           allow_raw: bool = False, out=None) -> CompressedTensor:
    """Compress a BF16 tensor of any shape through the flattened, block-padded layout.
    ``out``: optional placement of the result's tensors, see ``encode_components``."""
    if data.dtype != torch.bfloat16:
        raise TypeError(f"the codec compresses bfloat16 tensors, got {data.dtype}")
    shape = tuple(data.shape)
    source = data.contiguous().view(-1)
    logical_numel = source.numel()
    block_symbols, lanes, _, fixed_words = geometry(distribution)
    blocks = -(-logical_numel // block_symbols)
    storage_numel = blocks * block_symbols
    if allow_raw:
        # Keep the dense bytes when even an overflow-free encoding would be larger.
        smallest = storage_numel + (blocks * lanes * fixed_words + 4) * 4
        if smallest > logical_numel * data.element_size():
            return CompressedTensor(source, logical_numel, buffer=buffer, distribution=distribution,
                                    shape=shape, layout=StorageLayout.RAW)
    if out is None:
        sign_mantissa = torch.empty(storage_numel, dtype=torch.uint8, device=source.device)
    else:
        sign_mantissa = out.take("side", storage_numel, torch.uint8)
    return encode_components(
        source.view(torch.int16), sign_mantissa, storage_numel, distribution, buffer, shape,
        precomputed=False, logical_numel=logical_numel, out=out,
    )


# Result objects of ``encode_many(..., recycle=True)`` that were given back by
# ``operations.free_many(..., recycle=True)``, per (device, stream, arena, codebook, shape): the next
# compression of a tensor of that kind writes into the same storage, and the operand record
# cached with the object stays valid, so a layer that saves the same activations every step
# pays no allocation from its second step on.
_POOL_KEY = "_b200_pool_key"
_pool: dict = {}
MAX_POOLED = 4          # spare result objects kept per kind
MAX_POOL_KINDS = 64


def _pool_key(device, buffer, distribution, shape):
    index = device.index if device.index is not None else torch.cuda.current_device()
    return (index, dispatch._raw_stream(index), id(buffer), distribution.family, distribution.param,
            distribution.mean, distribution.zero_prob, distribution.noise_level, tuple(shape))


def give_back(items) -> None:
    """Make the storage of released results of ``encode_many(..., recycle=True)`` available to
    later calls.  The items must not be used afterwards."""
    for item in items:
        key = item.__dict__.get(_POOL_KEY)
        if key is None:
            continue
        spare = _pool.pop(key, [])
        if len(spare) < MAX_POOLED:
            spare.append(item)
        _pool[key] = spare                       # most recently used kind last
    while len(_pool) > MAX_POOL_KINDS:
        _pool.pop(next(iter(_pool)))


def forget_pooled_storage() -> None:
    _pool.clear()


def encode_many(tensors: list[torch.Tensor], distribution: Distribution,
                buffer: TensorBuffer, *, recycle: bool = False) -> list[CompressedTensor]:
    """Compress many BF16 tensors of any shapes with ONE codebook into ``buffer``'s arena by four
    launches in all (centers, encode, scans + reservations in list order, tails) instead of four
    per tensor.  Every result holds the tensors and the bytes ``encode`` gives it, and the arena
    ends up as after one ``encode`` per tensor in list order.  Nothing synchronises the host.
    No counterpart in the reference, which compresses one tensor per call
    (``LCT/codec/encode.py:189-218``); its layers do so for every activation they save.

    ``recycle``: take the results' storage from objects that ``free_many(..., recycle=True)``
    gave back (same arena, codebook and shape) instead of allocating it; for callers that own
    their compressed tensors exclusively and release them through that call."""
    if buffer is None:
        raise ValueError("encode_many needs a TensorBuffer")
    if buffer.capacity_bytes % 4:
        raise ValueError("TensorBuffer capacity must be divisible by 4")
    if not tensors:
        return []
    device = tensors[0].device
    stream_geometry = geometry(distribution)
    block_symbols, lanes, steps, fixed_words = stream_geometry
    encode_table, decode_table, _ = get_distribution_tables(distribution, device)

    def new(n, dtype):
        return torch.empty(n, dtype=dtype, device=device)

    results: list[CompressedTensor | None] = []
    jobs = []
    for data in tensors:
        if data.dtype != torch.bfloat16:
            raise TypeError(f"the codec compresses bfloat16 tensors, got {data.dtype}")
        if data.device != device:
            raise ValueError("encode_many needs all tensors on one device")
        if not data.numel():                 # nothing to launch: the one-tensor path's metadata
            results.append(encode(data, distribution, buffer))
            continue
        source = data.detach().contiguous().view(-1).view(torch.int16)
        blocks = -(-source.numel() // block_symbols)
        size = blocks * block_symbols
        key = _pool_key(device, buffer, distribution, data.shape) if recycle else None
        spare = _pool.get(key) if recycle else None
        if spare and spare[-1].buffer is buffer:
            c = spare.pop()
            jobs.append(dict(src=source, side=c.sign_mantissa, encoded=c.data, center=c.center,
                             decode_table=c.decode_table, counts=c.__dict__["_b200_counts"],
                             descriptor=c.fallback_descriptor, blocks=c.fallback_blocks,
                             size=size, logical_numel=source.numel()))
            results.append(c)
            continue
        counts = new(4, torch.int32)
        c = CompressedTensor(
            new(blocks * lanes * fixed_words + 4, torch.int32), size, new(size, torch.uint8),
            fallback_starts=None, fallback_lanes=None, fallback_blocks=new(3 * blocks, torch.int32),
            fallback_buffer=buffer.data, fallback_descriptor=new(4, torch.int32), buffer=buffer,
            fallback_count=counts[:1], fallback_used=counts[1:2], distribution=distribution,
            center=new(1, torch.int32), decode_table=new(decode_table.numel(), torch.int32),
            shape=tuple(data.shape), layout=StorageLayout.COMPRESSED,
            stream_geometry=stream_geometry)
        object.__setattr__(c, "_b200_counts", counts)
        if recycle:
            object.__setattr__(c, _POOL_KEY, key)
        jobs.append(dict(src=source, side=c.sign_mantissa, encoded=c.data, center=c.center,
                         decode_table=c.decode_table, counts=counts,
                         descriptor=c.fallback_descriptor, blocks=c.fallback_blocks, size=size,
                         logical_numel=source.numel()))
        results.append(c)
    if jobs:
        dispatch.compress_batch(jobs, encode_table, decode_table, buffer,
                                block_symbols=block_symbols, lanes=lanes, steps=steps,
                                fixed_words=fixed_words)
    return results
