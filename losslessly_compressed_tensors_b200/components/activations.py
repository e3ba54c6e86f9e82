"""Activations kept compressed between forward and backward.

The reference does this inside hand-written ``autograd.Function`` layers of its nanoGPT
example (``LCT/components/layers.py:22-305``, ``mlps.py``): each layer compresses the tensor
it needs for backward into one shared arena (``compress(x, distribution=act_dist,
buffer=buffer)`` when ``x.numel() >= min_elements``), and its backward decodes it and releases
the arena region.  Here the same ownership pattern is offered for ANY module, in two forms:

* ``ActivationCache`` - the explicit form: ``handle = cache.store(x)`` in a forward,
  ``x = handle.load()`` in the backward (decode, then the region goes back to the arena);
* ``compressed_saved_tensors(...)`` - a context manager over autograd's saved-tensor hooks that
  applies the cache to every eligible tensor the wrapped forward saves.

A cache built with ``batch=...`` compresses the tensors of a layer together (four launches
per group instead of four per tensor) and decodes them together (one launch).

Eligible: CUDA, bfloat16, at least ``min_elements`` elements, not a parameter (leaf that
requires grad).  Everything else is kept as it is.  The codec is lossless, so gradients are
bit-identical with and without the cache.
"""
from __future__ import annotations

import contextlib
import weakref

import torch
from torch import Tensor

from ..LCTensor import LCTTensor
from ..comp_format import Distribution
from ..operations import compress, compress_many, decompress, decompress_many, free_many
from ..tensor_buffer import TensorBuffer
from .dist_configs import act_dist, weight_dist


class _Group:
    """Tensors stored between two ``flush`` calls of a batching cache: compressed together by
    four launches, decoded together by one when the first of them is loaded, released together
    by one."""

    __slots__ = ("cache", "members")

    def __init__(self, cache: "ActivationCache"):
        self.cache, self.members = cache, []      # weak: a dropped graph must free its handles

    def add(self, handle: "_Handle") -> None:
        self.members.append(weakref.ref(handle))

    @property
    def handles(self) -> list:
        return [h for h in (ref() for ref in self.members) if h is not None]

    def compress(self) -> None:
        waiting = [h for h in self.handles if h._pending is not None]
        if not waiting:
            return
        results = compress_many([h._pending for h in waiting], self.cache.distribution,
                                self.cache.buffer, recycle=True)    # handles own them exclusively
        for handle, compressed in zip(waiting, results):
            handle._compressed, handle._pending = compressed, None

    def decode(self) -> None:
        held = [h for h in self.handles if h._compressed is not None]
        if not held:
            return
        for handle, dense in zip(held, decompress_many([h._compressed for h in held])):
            handle._dense = dense
        compressed = [h._compressed for h in held]
        for handle in held:
            handle._compressed = None
        free_many(compressed, recycle=True)


class _Handle:
    """One cached activation.  ``load`` may be called more than once (retained graphs); the
    compressed form is released at the first call and the dense tensor is kept from then on."""

    __slots__ = ("_compressed", "_dense", "_pending", "_group", "__weakref__")

    def __init__(self, compressed=None, dense=None, pending=None, group=None):
        self._compressed, self._dense, self._pending, self._group = compressed, dense, pending, group

    @property
    def is_compressed(self) -> bool:
        return self._compressed is not None

    def load(self) -> Tensor:
        if self._pending is not None:         # loaded before its group was compressed
            self._dense, self._pending = self._pending, None
        elif self._compressed is not None:
            if self._group is not None:
                self._group.decode()          # the whole group with one launch
            else:
                self._dense = decompress(self._compressed)
                self._compressed.free()
                self._compressed = None
        return self._dense

    def discard(self) -> None:
        """Release without decoding (a forward whose backward never runs)."""
        if self._compressed is not None:
            self._compressed.free()
            self._compressed = None
        self._dense = self._pending = None

    def __del__(self):
        # A graph dropped without a backward pass (an evaluation forward inside the context, an
        # exception between forward and backward) must give its arena regions back.
        try:
            self.discard()
        except Exception:       # interpreter shutdown: the CUDA context may be gone already
            pass


class ActivationCache:
    """Stores eligible tensors compressed in ``buffer`` (or in private tensors without one).

    ``batch``: collect that many eligible tensors (or all until ``flush()``, with ``batch=0``)
    and compress them together - four launches per group instead of four per tensor; the first
    ``load`` of a group member decodes the whole group with one launch and releases its regions
    with one more.  A layer's activations are saved together and needed together, so a group
    per layer (``flush()`` at each layer's end, or ``batch`` = tensors saved per layer) costs
    no extra peak memory.  Until a group is compressed its tensors are kept dense.  Needs a
    ``buffer``.  ``batch=None`` (default): every tensor is compressed on its own at once."""

    def __init__(self, buffer: TensorBuffer | None = None, distribution: Distribution | None = None,
                 min_elements: int = 65536, batch: int | None = None):
        if batch is not None and buffer is None:
            raise ValueError("a batching ActivationCache needs a TensorBuffer")
        self.buffer = buffer
        self.distribution = distribution or act_dist
        self.min_elements = int(min_elements)
        self.batch = batch
        self._group = _Group(self) if batch is not None else None
        self.stored = 0           # tensors compressed (or queued for it) so far
        self.dense_bytes = 0      # their BF16 bytes
        self.compressed_bytes = 0

    def eligible(self, tensor: Tensor) -> bool:
        return (tensor.device.type == "cuda" and tensor.dtype == torch.bfloat16
                and tensor.numel() >= self.min_elements
                and not (tensor.is_leaf and tensor.requires_grad)
                and not isinstance(tensor, LCTTensor))

    def store(self, tensor: Tensor, *, track_sizes: bool = False) -> _Handle:
        if not self.eligible(tensor):
            return _Handle(dense=tensor)
        self.stored += 1
        if self._group is not None:
            handle = _Handle(pending=tensor.detach(), group=self._group)
            self._group.add(handle)
            if self.batch and len(self._group.members) >= self.batch:
                self.flush()
            return handle
        compressed = compress(tensor.detach(), distribution=self.distribution, buffer=self.buffer)
        if track_sizes:   # memory_size() reads device counters: a host synchronisation
            self.dense_bytes += tensor.numel() * 2
            self.compressed_bytes += compressed.memory_size()
        return _Handle(compressed=compressed)

    def flush(self) -> None:
        """Compress the tensors stored since the last flush as one group and start a new one."""
        if self._group is not None and self._group.members:
            self._group.compress()
            self._group = _Group(self)


@contextlib.contextmanager
def compressed_saved_tensors(buffer: TensorBuffer | None = None,
                             distribution: Distribution | None = None, min_elements: int = 65536,
                             cache: ActivationCache | None = None):
    """Within the block, tensors that autograd saves for backward go through an
    ``ActivationCache`` (yielded, for its counters)."""
    cache = cache or ActivationCache(buffer, distribution, min_elements)
    try:
        with torch.autograd.graph.saved_tensors_hooks(cache.store, _Handle.load):
            yield cache
    finally:
        cache.flush()      # a batching cache: what the forward stored last


def dense_weight(weight: Tensor) -> Tensor:
    """The BF16 values of a weight that may be stored compressed (``layers.py:12-13``)."""
    return weight.decompress() if isinstance(weight, LCTTensor) else weight


def compress_weight(module: torch.nn.Module, buffer: TensorBuffer | None = None,
                    distribution: Distribution | None = None) -> None:
    """Replace ``module.weight`` (BF16) by its compressed form, once, after initialisation and
    checkpoint loading (``layers.py:289-295``)."""
    if isinstance(module.weight, LCTTensor):
        return
    packed = LCTTensor(module.weight.detach(), buffer=buffer, dist=distribution or weight_dist)
    del module._parameters["weight"]
    module.weight = packed
