"""Weight sets compressed across the GPUs of one node: partition, wire format, all-gather, decode.

The codec shards by construction: every tensor - and every row-shard of a tensor, compressed as a
tensor of its own with its own center and padding - is independent.  Ranks therefore encode
disjoint shards with no communication, and the only exchange is ONE ``all_gather_into_tensor`` of
the compressed bytes (about 0.70x of the dense BF16 bytes cross NVLink), after which every rank
decodes all shards from its local copy of the gathered buffer.

No size negotiation and no host synchronisation: the wire size of a shard follows from its shape
alone.  A rank's wire buffer is::

    [ shard 0: center | counts | descriptor | decode table | block metadata | payload | side bytes ]
    [ shard 1: ... ] ... [ arena: allocator words | overflow payload (fixed capacity) ]

Overflow tails of all of a rank's shards go to that rank's arena (a ``TensorBuffer`` living inside
the wire buffer); their descriptors travel in the shard headers.  Buffers are padded to the
largest rank so the collective is a plain equal-size all-gather.  The encoder writes its results
straight into the wire buffer (``encode(..., out=...)``), so packing costs no extra copy.

The reference has no distributed code at all; the names here are this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .codec.geometry import geometry
from .comp_format import Distribution, StorageLayout
from .comp_tensor import CompressedTensor

_ALIGN = 256
_DECODE_TABLE_WORDS = 1024
_FIELDS = ("center", "counts", "descriptor", "decode_table", "blocks", "encoded", "side")


def _up(n: int) -> int:
    return -(-n // _ALIGN) * _ALIGN


@dataclass(frozen=True)
class Shard:
    """A contiguous run of rows of one named tensor, compressed as an independent tensor."""

    name: str
    index: int              # position of the tensor in the weight set
    row_start: int
    row_stop: int
    shape: tuple[int, ...]  # shape of the shard itself

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass
class Plan:
    """Which rank encodes which shard, and where everything sits on the wire."""

    world: int
    distribution: Distribution
    shards: list[list[Shard]]                       # per rank, in wire order
    arena_capacity: int
    max_free_regions: int
    offsets: list[list[dict[str, tuple[int, int]]]] = field(default_factory=list)
    arena_offset: list[int] = field(default_factory=list)
    wire_bytes: int = 0

    def shard_blocks(self, shard: Shard) -> int:
        block_symbols = geometry(self.distribution)[0]
        return -(-shard.numel // block_symbols)


def split_rows(name: str, index: int, shape: tuple[int, ...], max_elements: int) -> list[Shard]:
    """Cut a tensor into row-shards of at most ``max_elements`` elements (whole rows)."""
    shape = tuple(int(d) for d in shape)
    numel = 1
    for d in shape:
        numel *= d
    rows = shape[0] if shape else 1
    if not shape or numel <= max_elements or rows <= 1:
        return [Shard(name, index, 0, rows, shape)]
    row_elements = numel // rows
    rows_per_shard = max(1, max_elements // row_elements)
    out = []
    for start in range(0, rows, rows_per_shard):
        stop = min(rows, start + rows_per_shard)
        out.append(Shard(name, index, start, stop, (stop - start,) + shape[1:]))
    return out


def make_plan(named_shapes: list[tuple[str, tuple[int, ...]]], world: int,
              distribution: Distribution, *, row_shard_elements: int | None = None,
              arena_fraction: float = 1.0 / 64, max_free_regions: int = 256) -> Plan:
    """Greedy longest-first assignment of shards to ranks; deterministic on every rank.

    ``row_shard_elements``: tensors larger than this are cut into row-shards first (``None``
    keeps tensors whole, i.e. per-tensor sharding).  ``arena_fraction``: overflow capacity of a
    rank as a fraction of its dense bytes (at least 64 KiB).
    """
    if world < 1:
        raise ValueError("world must be positive")
    pieces: list[Shard] = []
    for index, (name, shape) in enumerate(named_shapes):
        limit = row_shard_elements if row_shard_elements else 1 << 62
        pieces.extend(split_rows(name, index, tuple(shape), limit))
    # A shard costs whole codec blocks, however few elements it has.
    block_symbols = geometry(distribution)[0]
    cost = [-(-piece.numel // block_symbols) * block_symbols for piece in pieces]
    order = sorted(range(len(pieces)), key=lambda i: (-cost[i], i))
    load = [0] * world
    assigned: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        rank = min(range(world), key=lambda r: (load[r], r))
        assigned[rank].append(i)
        load[rank] += cost[i]
    shards = [[pieces[i] for i in sorted(ids)] for ids in assigned]
    capacity = max(64 << 10, int(max(load) * 2 * arena_fraction))
    capacity = -(-capacity // 16) * 16
    plan = Plan(world, distribution, shards, capacity, max_free_regions)
    _lay_out(plan)
    return plan


def _field_bytes(plan: Plan, shard: Shard) -> dict[str, int]:
    block_symbols, lanes, _, fixed_words = geometry(plan.distribution)
    blocks = plan.shard_blocks(shard)
    return {
        "center": 4, "counts": 16, "descriptor": 16, "decode_table": 4 * _DECODE_TABLE_WORDS,
        "blocks": 12 * blocks, "encoded": 4 * (blocks * lanes * fixed_words + 4),
        "side": blocks * block_symbols,
    }


def _lay_out(plan: Plan) -> None:
    from .tensor_buffer import TensorBuffer

    arena_bytes = TensorBuffer.storage_bytes(plan.arena_capacity, plan.max_free_regions)
    plan.offsets, plan.arena_offset, sizes = [], [], []
    for rank_shards in plan.shards:
        cursor, per_rank = 0, []
        for shard in rank_shards:
            slots = {}
            for name, nbytes in _field_bytes(plan, shard).items():
                slots[name] = (cursor, nbytes)
                cursor += _up(nbytes)
            per_rank.append(slots)
        plan.offsets.append(per_rank)
        plan.arena_offset.append(cursor)
        sizes.append(cursor + _up(arena_bytes))
    plan.wire_bytes = max(sizes)


_DTYPES = {"center": torch.int32, "counts": torch.int32, "descriptor": torch.int32,
           "decode_table": torch.int32, "blocks": torch.int32, "encoded": torch.int32,
           "side": torch.uint8}


def _slot(wire: torch.Tensor, slot: tuple[int, int], name: str) -> torch.Tensor:
    start, nbytes = slot
    return wire[start:start + nbytes].view(_DTYPES[name])


class _Placement:
    """``out=`` object for ``encode``: hands out the slots of one shard."""

    def __init__(self, wire: torch.Tensor, slots: dict[str, tuple[int, int]]):
        self.wire, self.slots = wire, slots

    def take(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        view = _slot(self.wire, self.slots[name], name)
        if view.dtype != dtype or view.numel() != numel:
            raise RuntimeError(f"wire slot {name!r} does not match the encoder's request")
        return view


def shard_source(tensors: list[torch.Tensor], shard: Shard) -> torch.Tensor:
    """The rows of the weight set that ``shard`` covers (a view when the tensor is contiguous)."""
    tensor = tensors[shard.index]
    if tensor.dim() == 0:
        return tensor.reshape(())
    return tensor[shard.row_start:shard.row_stop]


def encode_rank(plan: Plan, rank: int, tensors: list[torch.Tensor],
                wire: torch.Tensor | None = None):
    """Compress this rank's shards straight into its wire buffer.

    Returns ``(wire, compressed, arena)``: the uint8 buffer of ``plan.wire_bytes`` bytes, the
    ``CompressedTensor`` of every shard (their tensors are views of ``wire``) and the rank's
    ``TensorBuffer``.  Nothing here synchronises the host.
    """
    from .operations import compress
    from .tensor_buffer import TensorBuffer

    device = tensors[0].device if tensors else torch.device("cuda")
    if wire is None:
        wire = torch.zeros(plan.wire_bytes, dtype=torch.uint8, device=device)
    elif wire.numel() != plan.wire_bytes or wire.dtype != torch.uint8:
        raise ValueError("wire buffer has the wrong size or dtype")
    start = plan.arena_offset[rank]
    arena_bytes = TensorBuffer.storage_bytes(plan.arena_capacity, plan.max_free_regions)
    arena = TensorBuffer(plan.arena_capacity, max_free_regions=plan.max_free_regions,
                         storage=wire[start:start + arena_bytes])
    compressed = []
    for shard, slots in zip(plan.shards[rank], plan.offsets[rank]):
        source = shard_source(tensors, shard)
        if tuple(source.shape) != shard.shape:
            raise ValueError(f"{shard.name}: expected shape {shard.shape}, got {tuple(source.shape)}")
        from .codec.encode import encode

        compressed.append(encode(source.detach(), plan.distribution, arena,
                                 out=_Placement(wire, slots)))
    return wire, compressed, arena


def all_gather_wire(wire: torch.Tensor, plan: Plan, group=None) -> torch.Tensor:
    """The one collective of the path: every rank receives every rank's wire buffer."""
    import torch.distributed as dist

    gathered = torch.empty(plan.world * plan.wire_bytes, dtype=torch.uint8, device=wire.device)
    if plan.world == 1:
        gathered.copy_(wire)
    else:
        if dist.get_world_size(group) != plan.world:
            raise ValueError("plan was made for a different number of ranks")
        dist.all_gather_into_tensor(gathered, wire, group=group)
    return gathered


def views_of(plan: Plan, gathered: torch.Tensor) -> list[tuple[Shard, CompressedTensor]]:
    """Rebuild a ``CompressedTensor`` for every shard of every rank as views of ``gathered``."""
    from .tensor_buffer import TensorBuffer

    if gathered.numel() != plan.world * plan.wire_bytes:
        raise ValueError("gathered buffer has the wrong size")
    stream_geometry = geometry(plan.distribution)
    block_symbols = stream_geometry[0]
    metadata = TensorBuffer.storage_bytes(0, plan.max_free_regions)
    result = []
    for rank in range(plan.world):
        wire = gathered[rank * plan.wire_bytes:(rank + 1) * plan.wire_bytes]
        arena_start = plan.arena_offset[rank] + metadata
        arena_payload = wire[arena_start:arena_start + plan.arena_capacity]
        for shard, slots in zip(plan.shards[rank], plan.offsets[rank]):
            counts = _slot(wire, slots["counts"], "counts")
            result.append((shard, CompressedTensor(
                _slot(wire, slots["encoded"], "encoded"),
                plan.shard_blocks(shard) * block_symbols,
                _slot(wire, slots["side"], "side"),
                fallback_blocks=_slot(wire, slots["blocks"], "blocks"),
                fallback_buffer=arena_payload,
                fallback_descriptor=_slot(wire, slots["descriptor"], "descriptor"),
                fallback_count=counts[:1], fallback_used=counts[1:2],
                distribution=plan.distribution, center=_slot(wire, slots["center"], "center"),
                decode_table=_slot(wire, slots["decode_table"], "decode_table"),
                shape=shard.shape, layout=StorageLayout.COMPRESSED,
                stream_geometry=stream_geometry,
            )))
    return result


def decode_all(plan: Plan, gathered: torch.Tensor, shapes: list[tuple[int, ...]]):
    """Decode every shard from the gathered bytes and reassemble the weight set."""
    from .operations import decompress

    outputs = [torch.empty(shape, dtype=torch.bfloat16, device=gathered.device) for shape in shapes]
    for shard, compressed in views_of(plan, gathered):
        dense = decompress(compressed)
        target = outputs[shard.index]
        if target.dim() == 0:
            target.copy_(dense.reshape(()))
        else:
            target[shard.row_start:shard.row_stop].copy_(dense)
    return outputs


def gpt2_small_shapes(layers: int = 12, d_model: int = 768, vocab: int = 50304,
                      context: int = 1024) -> list[tuple[str, tuple[int, ...]]]:
    """The 148 tensors (124 475 904 parameters) of a GPT-2-small-shaped weight set, tied head."""
    shapes = [("wte", (vocab, d_model)), ("wpe", (context, d_model))]
    for i in range(layers):
        p = f"h.{i}."
        shapes += [
            (p + "ln_1.weight", (d_model,)), (p + "ln_1.bias", (d_model,)),
            (p + "attn.c_attn.weight", (d_model, 3 * d_model)), (p + "attn.c_attn.bias", (3 * d_model,)),
            (p + "attn.c_proj.weight", (d_model, d_model)), (p + "attn.c_proj.bias", (d_model,)),
            (p + "ln_2.weight", (d_model,)), (p + "ln_2.bias", (d_model,)),
            (p + "mlp.c_fc.weight", (d_model, 4 * d_model)), (p + "mlp.c_fc.bias", (4 * d_model,)),
            (p + "mlp.c_proj.weight", (4 * d_model, d_model)), (p + "mlp.c_proj.bias", (d_model,)),
        ]
    shapes += [("ln_f.weight", (d_model,)), ("ln_f.bias", (d_model,))]
    return shapes
