"""Device-resident first-fit arena shared by the overflow tails of many tensors.

API and memory layout of the reference's ``TensorBuffer`` (``LCT/tensor_buffer.py:13-201``):
one uint8 tensor holding ``free_starts[R] | free_sizes[R] | free_count | lock |
generation | pad | payload[capacity]``; requests and results stay on the device as
``[offset, aligned_size, status, generation]`` descriptors, so allocating and
freeing never synchronise the host.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .kernels import dispatch

_ALIGNMENT = 16


@dataclass(frozen=True)
class Allocation:
    """A device ``[offset, aligned_size, status, generation]`` descriptor and its arena.
    ``offset``, ``size``, ``status`` and ``generation`` are 0-dim views of the four words
    (reading their values synchronises; handing them to kernels does not)."""

    descriptor: torch.Tensor
    owner: object


def _descriptor_word(index: int, name: str) -> property:
    def read(self: Allocation) -> torch.Tensor:
        return self.descriptor[index]

    read.__name__ = name
    return property(read)


for _index, _name in enumerate(("offset", "size", "status", "generation")):
    setattr(Allocation, _name, _descriptor_word(_index, _name))
del _index, _name


@torch.library.custom_op("lct::tensor_buffer_free", mutates_args=("storage", "descriptor"))
def tensor_buffer_free(storage: torch.Tensor, descriptor: torch.Tensor,
                       max_free_regions: int) -> torch.Tensor:
    """Opaque to ``torch.compile`` like the reference's op (``LCT/kernels/tensor_buffer_ops.py:5-20``)."""
    status = torch.empty(1, dtype=torch.int32, device=storage.device)
    dispatch.buffer_free(storage, descriptor, status, max_free_regions)
    return status


@tensor_buffer_free.register_fake
def _tensor_buffer_free_fake(storage, descriptor, max_free_regions):
    return torch.empty(1, dtype=torch.int32, device=storage.device)


class TensorBuffer:
    """First-fit allocator living in device memory.

    ``max_free_regions`` bounds the free list (a power of two).  Callers hand the
    payload tensor (``data``) and the device descriptors straight to kernels.
    """

    def __init__(self, capacity_bytes: int, *, max_free_regions: int = 256,
                 device: torch.device | str | None = None,
                 storage: torch.Tensor | None = None) -> None:
        """``storage`` (not in the reference): build the arena inside an existing uint8 tensor of
        ``storage_bytes(capacity_bytes, max_free_regions)`` bytes, e.g. a slice of a wire buffer."""
        if capacity_bytes > torch.iinfo(torch.int32).max:
            raise ValueError("capacity_bytes must fit in int32")
        if max_free_regions <= 0 or max_free_regions & (max_free_regions - 1):
            raise ValueError("max_free_regions must be a positive power of two")
        self.capacity_bytes = int(capacity_bytes)
        self.max_free_regions = int(max_free_regions)
        regions = self.max_free_regions
        self._metadata_bytes = self._align(8 * regions + 12)
        if storage is None:
            self._storage = torch.zeros(self._metadata_bytes + self.capacity_bytes,
                                        dtype=torch.uint8, device=torch.device(device or "cuda"))
        else:
            if (storage.dtype != torch.uint8 or storage.dim() != 1 or not storage.is_contiguous()
                    or storage.numel() != self._metadata_bytes + self.capacity_bytes
                    or storage.data_ptr() % _ALIGNMENT):
                raise ValueError("storage must be a contiguous, 16-byte aligned uint8 tensor of "
                                 "storage_bytes(capacity_bytes, max_free_regions) bytes")
            self._storage = storage
            self._storage[: self._metadata_bytes].zero_()
        self.device = self._storage.device
        words = self._storage[: 8 * regions + 12].view(torch.int32)
        self._free_starts = words[:regions]
        self._free_sizes = words[regions: 2 * regions]
        self._free_count = words[2 * regions: 2 * regions + 1]
        self._lock = words[2 * regions + 1: 2 * regions + 2]
        self._generation = words[2 * regions + 2: 2 * regions + 3]
        self._data = self._storage[self._metadata_bytes:]
        self.reset()

    @staticmethod
    def _align(nbytes: int) -> int:
        return -(-nbytes // _ALIGNMENT) * _ALIGNMENT

    @classmethod
    def storage_bytes(cls, capacity_bytes: int, max_free_regions: int = 256) -> int:
        """Bytes of the backing tensor: allocator words, padding, then the payload."""
        return cls._align(8 * max_free_regions + 12) + int(capacity_bytes)

    @property
    def data(self) -> torch.Tensor:
        """The payload bytes descriptors index into."""
        return self._data

    def _request(self, value: torch.Tensor) -> torch.Tensor:
        value = value.reshape(-1)[:1]
        if value.dtype != torch.int32 or value.device != self.device:
            value = value.to(device=self.device, dtype=torch.int32)
        return value

    def allocate(self, nbytes: torch.Tensor) -> Allocation:
        """Reserve ``nbytes`` (a one-element device integer tensor) without a host sync."""
        descriptor = torch.empty(4, dtype=torch.int32, device=self.device)
        dispatch.buffer_allocate(self._storage, self._request(nbytes), None, 0, descriptor,
                                 self.max_free_regions)
        return Allocation(descriptor, self)

    def allocate_with_items(self, payload_bytes: torch.Tensor, item_count: torch.Tensor,
                            item_bytes: int) -> Allocation:
        """Reserve ``payload_bytes + item_count * item_bytes``, both read on the device."""
        if item_bytes <= 0:
            raise ValueError("item_bytes must be positive")
        descriptor = torch.empty(4, dtype=torch.int32, device=self.device)
        dispatch.buffer_allocate(self._storage, self._request(payload_bytes),
                                 self._request(item_count), int(item_bytes), descriptor,
                                 self.max_free_regions)
        return Allocation(descriptor, self)

    def free(self, allocation: Allocation) -> torch.Tensor:
        """Return a region; the result is a device status word (0 ok, 3 list full, 4 stale/invalid)."""
        if allocation.owner is not self:
            raise ValueError("allocation belongs to a different allocator")
        if allocation.descriptor.device != self.device:
            raise ValueError("allocation must be on the allocator device")
        if torch.compiler.is_compiling():
            return tensor_buffer_free(self._storage, allocation.descriptor, self.max_free_regions)
        # Eager mode: the same launch without the operator dispatcher in between.
        status = torch.empty(1, dtype=torch.int32, device=self.device)
        dispatch.buffer_free(self._storage, allocation.descriptor, status, self.max_free_regions)
        return status

    def free_many(self, descriptors: list[torch.Tensor]) -> torch.Tensor:
        """Return many regions with one launch, in list order (the free list ends up as after
        one ``free`` each); the result holds one status word per descriptor."""
        status = torch.empty(max(1, len(descriptors)), dtype=torch.int32, device=self.device)
        if descriptors:
            pointers = torch.empty(len(descriptors), dtype=torch.int64, pin_memory=True)
            pointers.copy_(torch.tensor([d.data_ptr() for d in descriptors], dtype=torch.int64))
            table = pointers.to(self.device, non_blocking=True)     # asynchronous: pinned source
            dispatch._call("lct_buffer_free_many", self.device, self._storage.data_ptr(),
                           table.data_ptr(), len(descriptors), status.data_ptr(),
                           self.max_free_regions)
            self._keep = (table, descriptors)      # until the next call: the launch reads them
        return status

    def reset(self) -> None:
        """Forget every allocation; outstanding descriptors become stale (generation bump)."""
        dispatch.buffer_reset(self._storage, self.max_free_regions, self.capacity_bytes)


def _free_regions_snapshot(buffer: TensorBuffer) -> list[tuple[int, int]]:
    """Synchronise and return the free list as ``(start, size)`` pairs."""
    regions = buffer.max_free_regions
    words = buffer._storage[: buffer._metadata_bytes].view(torch.int32).cpu().tolist()
    count = words[2 * regions]
    if not 0 <= count <= regions:
        raise RuntimeError(f"corrupt free-list count: {count}")
    return [(words[i], words[regions + i]) for i in range(count)]


def verify_buffer(buffer: TensorBuffer) -> None:
    """Synchronise and check the free list: regions sorted, inside the payload, non-empty, and
    no two of them touching (a free must have merged them)."""
    regions = _free_regions_snapshot(buffer)
    cursor = 0
    for index, (start, size) in enumerate(regions):
        stop = start + size
        if size <= 0 or start < cursor or stop > buffer.capacity_bytes:
            raise RuntimeError(f"invalid free region: [{start}, {stop})")
        if index and start == cursor:
            raise RuntimeError("adjacent free regions were not coalesced")
        cursor = stop
    if sum(size for _, size in regions) > buffer.capacity_bytes:
        raise RuntimeError("free regions exceed payload capacity")


def visualize_buffer(buffer: TensorBuffer | None, width: int = 80) -> str:
    """Synchronise and draw the payload as a strip of ``width`` cells: ``#`` where bytes are in
    use, ``.`` where a cell touches a free region, followed by the free list."""
    if buffer is None:
        return ""
    if width < 8:
        raise ValueError("width must be at least 8")
    capacity = buffer.capacity_bytes
    free = _free_regions_snapshot(buffer)
    strip = bytearray(b"#" * width)
    for start, size in free:
        first = start * width // capacity
        past = -(-(start + size) * width // capacity)          # ceiling
        for cell in range(first, min(width, max(first + 1, past))):
            strip[cell] = ord(".")
    in_use = capacity - sum(size for _, size in free)
    listed = [f"[{start}, {start + size})" for start, size in free]
    if len(listed) > 8:
        listed[4:-4] = ["..."]
    return "\n".join((
        f"arena payload {in_use} of {capacity} B in use ({in_use / capacity:.1%}), "
        f"{len(free)} free region(s)",
        f"0 |{strip.decode()}| {capacity}",
        "legend: # in use, . free",
        "free regions: " + (", ".join(listed) if listed else "none"),
    ))
