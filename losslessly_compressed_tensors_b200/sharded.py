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
    # Prepared launches, keyed by the addresses AND layouts they were prepared for: a training
    # loop that re-encodes the same parameters into the same wire buffer every step pays the
    # Python cost of describing 150+ shards once.  A prepared launch keeps its tensors alive, so
    # only launches on caller-owned, reusable buffers are kept, and only the most recent few.
    prepared: dict = field(default_factory=dict, repr=False, compare=False)
    max_prepared: int = 8

    def remember(self, key, value) -> None:
        """Keep a prepared launch; the oldest entries go once ``max_prepared`` are held."""
        self.prepared.pop(key, None)
        self.prepared[key] = value
        while len(self.prepared) > self.max_prepared:
            self.prepared.pop(next(iter(self.prepared)))

    def recall(self, key):
        hit = self.prepared.pop(key, None)
        if hit is not None:
            self.prepared[key] = hit     # most recently used last
        return hit

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


def _identity(t: torch.Tensor) -> tuple:
    """What a prepared launch depends on: where a tensor lives and how it is laid out."""
    return (t.data_ptr(), tuple(t.shape), t.dtype, tuple(t.stride()))


def shard_source(tensors: list[torch.Tensor], shard: Shard) -> torch.Tensor:
    """The rows of the weight set that ``shard`` covers (a view when the tensor is contiguous)."""
    tensor = tensors[shard.index]
    if tensor.dim() == 0:
        return tensor.reshape(())
    return tensor[shard.row_start:shard.row_stop]


def _compressed_view(plan: Plan, wire: torch.Tensor, shard: Shard, slots, arena_payload,
                     buffer=None) -> CompressedTensor:
    """The ``CompressedTensor`` whose tensors are the wire slots of one shard."""
    stream_geometry = geometry(plan.distribution)
    counts = _slot(wire, slots["counts"], "counts")
    return CompressedTensor(
        _slot(wire, slots["encoded"], "encoded"),
        plan.shard_blocks(shard) * stream_geometry[0],
        _slot(wire, slots["side"], "side"),
        fallback_blocks=_slot(wire, slots["blocks"], "blocks"),
        fallback_buffer=arena_payload,
        fallback_descriptor=_slot(wire, slots["descriptor"], "descriptor"),
        buffer=buffer,
        fallback_count=counts[:1], fallback_used=counts[1:2],
        distribution=plan.distribution, center=_slot(wire, slots["center"], "center"),
        decode_table=_slot(wire, slots["decode_table"], "decode_table"),
        shape=shard.shape, layout=StorageLayout.COMPRESSED, stream_geometry=stream_geometry,
    )


def encode_rank(plan: Plan, rank: int, tensors: list[torch.Tensor],
                wire: torch.Tensor | None = None, *, batched: bool = True):
    """Compress this rank's shards straight into its wire buffer.

    Returns ``(wire, compressed, arena)``: the uint8 buffer of ``plan.wire_bytes`` bytes, the
    ``CompressedTensor`` of every shard (their tensors are views of ``wire``) and the rank's
    ``TensorBuffer``.  ``batched`` encodes all shards with four launches in total instead of
    four per shard; the bytes are the same.  Nothing here synchronises the host.
    """
    from .codec.encode import encode
    from .compression.huffman_tables import get_distribution_tables
    from .kernels import dispatch
    from .tensor_buffer import TensorBuffer

    device = tensors[0].device if tensors else torch.device("cuda")
    caller_owns_wire = wire is not None
    if wire is None:
        wire = torch.zeros(plan.wire_bytes, dtype=torch.uint8, device=device)
    elif wire.numel() != plan.wire_bytes or wire.dtype != torch.uint8:
        raise ValueError("wire buffer has the wrong size or dtype")
    key = ("encode", rank, batched, wire.data_ptr(), tuple(_identity(t) for t in tensors))
    hit = plan.recall(key) if caller_owns_wire else None
    if hit is not None and batched:
        batch, compressed, arena, metadata_bytes = hit
        arena._storage[:metadata_bytes].zero_()   # same state as a freshly built arena
        arena.reset()
        batch.run()
        return wire, compressed, arena
    start = plan.arena_offset[rank]
    arena_bytes = TensorBuffer.storage_bytes(plan.arena_capacity, plan.max_free_regions)
    arena = TensorBuffer(plan.arena_capacity, max_free_regions=plan.max_free_regions,
                         storage=wire[start:start + arena_bytes])
    sources = []
    for shard in plan.shards[rank]:
        source = shard_source(tensors, shard)
        if tuple(source.shape) != shard.shape:
            raise ValueError(f"{shard.name}: expected shape {shard.shape}, got {tuple(source.shape)}")
        if source.dtype != torch.bfloat16:
            raise TypeError(f"{shard.name}: the codec compresses bfloat16 tensors")
        sources.append(source.detach())
    if not batched or not sources:
        compressed = [encode(source, plan.distribution, arena, out=_Placement(wire, slots))
                      for source, slots in zip(sources, plan.offsets[rank])]
        return wire, compressed, arena

    block_symbols, lanes, steps, fixed_words = geometry(plan.distribution)
    encode_table, decode_table, _ = get_distribution_tables(plan.distribution, device)
    compressed, jobs = [], []
    for shard, source, slots in zip(plan.shards[rank], sources, plan.offsets[rank]):
        c = _compressed_view(plan, wire, shard, slots, arena.data, arena)
        flat = source.contiguous().view(-1).view(torch.int16)
        jobs.append(dict(src=flat, side=c.sign_mantissa, encoded=c.data, center=c.center,
                         decode_table=c.decode_table, counts=c.fallback_count,
                         descriptor=c.fallback_descriptor, blocks=c.fallback_blocks,
                         size=c.size, logical_numel=flat.numel()))
        compressed.append(c)
    batch = dispatch.compress_batch(jobs, encode_table, decode_table, arena,
                                    block_symbols=block_symbols, lanes=lanes, steps=steps,
                                    fixed_words=fixed_words)
    if caller_owns_wire and all(job["src"].data_ptr() == shard_source(tensors, shard).data_ptr()
                                for job, shard in zip(jobs, plan.shards[rank])):   # no temporaries
        plan.remember(key, (batch, compressed, arena,
                            TensorBuffer.storage_bytes(0, plan.max_free_regions)))
    return wire, compressed, arena


def all_gather_wire(wire: torch.Tensor, plan: Plan, group=None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """The one collective of the path: every rank receives every rank's wire buffer.
    ``out`` reuses a previous result buffer (and with it the prepared decode launch)."""
    import torch.distributed as dist

    gathered = out if out is not None else torch.empty(
        plan.world * plan.wire_bytes, dtype=torch.uint8, device=wire.device)
    if gathered.numel() != plan.world * plan.wire_bytes:
        raise ValueError("gathered buffer has the wrong size")
    if plan.world == 1:
        gathered.copy_(wire)
    else:
        if dist.get_world_size(group) != plan.world:
            raise ValueError("plan was made for a different number of ranks")
        dist.all_gather_into_tensor(gathered, wire, group=group)
    return gathered


def _wires_of(plan: Plan, gathered) -> list[torch.Tensor]:
    """Per-rank wire buffers from either one gathered buffer or a list of (peer) buffers."""
    if isinstance(gathered, (list, tuple)):
        if len(gathered) != plan.world or any(w.numel() != plan.wire_bytes for w in gathered):
            raise ValueError("expected one wire buffer of plan.wire_bytes per rank")
        return list(gathered)
    if gathered.numel() != plan.world * plan.wire_bytes:
        raise ValueError("gathered buffer has the wrong size")
    return [gathered[rank * plan.wire_bytes:(rank + 1) * plan.wire_bytes] for rank in range(plan.world)]


def views_of(plan: Plan, gathered) -> list[tuple[Shard, CompressedTensor]]:
    """Rebuild a ``CompressedTensor`` for every shard of every rank as views of the wire bytes:
    ``gathered`` is the all-gathered buffer, or a list with every rank's wire buffer (which may
    live in peer GPUs' memory, see ``PeerWire``).  Rank-major order."""
    return [(shard, compressed) for _, shard, compressed in _views_with_rank(plan, gathered)]


def _views_with_rank(plan: Plan, gathered) -> list[tuple[int, Shard, CompressedTensor]]:
    from .tensor_buffer import TensorBuffer

    metadata = TensorBuffer.storage_bytes(0, plan.max_free_regions)
    result = []
    for rank, wire in enumerate(_wires_of(plan, gathered)):
        arena_start = plan.arena_offset[rank] + metadata
        arena_payload = wire[arena_start:arena_start + plan.arena_capacity]
        for shard, slots in zip(plan.shards[rank], plan.offsets[rank]):
            result.append((rank, shard, _compressed_view(plan, wire, shard, slots, arena_payload)))
    return result


def check(plan: Plan, gathered) -> None:
    """Raise if any shard of any rank lost its overflow tails.

    Encoding never synchronises the host, so a rank whose arena was too small (or whose
    allocator gave up) only records that in the shard's descriptor: status 0 = stored.  A decode
    of such a shard would silently leave its overflow lanes' tails undecoded.  This reads every
    descriptor and overflow count of the gathered wire in one device-to-host copy; call it once
    after the first exchange of a new weight set (or every step, at the price of a
    synchronisation) and raise ``arena_fraction`` in ``make_plan`` when it fires."""
    views = _views_with_rank(plan, gathered)
    if not views:
        return
    words = torch.stack([torch.cat((c.fallback_descriptor[:3].to(views[0][2].data.device),
                                    c.fallback_count.to(views[0][2].data.device)))
                         for _, _, c in views]).cpu().tolist()
    lost = [f"rank {rank} {shard.name}[{shard.row_start}:{shard.row_stop}] status {status} "
            f"({count} overflow streams)"
            for (rank, shard, _), (_, _, status, count) in zip(views, words)
            if status != 0 and count > 0]
    if lost:
        raise RuntimeError("overflow tails were not stored (arena too small for this weight set: "
                           "raise arena_fraction): " + "; ".join(lost[:8])
                           + (f" and {len(lost) - 8} more" if len(lost) > 8 else ""))


def _interleaved(plan: Plan, views: list, first_rank: int) -> list:
    """Reorder rank-major (shard, tensor) pairs round-robin over the source ranks, starting at
    ``first_rank``: consecutive CTAs of a decode launch then read from different sources, and
    when every rank starts one source further on, no source serves all readers at once."""
    per_rank, at = [], 0
    for rank in range(plan.world):
        count = len(plan.shards[rank])
        per_rank.append(views[at:at + count])
        at += count
    order = [(first_rank + k) % plan.world for k in range(plan.world)]
    out = []
    for k in range(max(len(v) for v in per_rank)):
        out.extend(per_rank[r][k] for r in order if k < len(per_rank[r]))
    return out


def decode_all(plan: Plan, gathered, shapes: list[tuple[int, ...]], *, batched: bool = True,
               outputs: list[torch.Tensor] | None = None, interleave_from: int | None = None,
               stage_remote_for: int | None = None):
    """Decode every shard from the wire bytes and reassemble the weight set.  ``gathered``: the
    all-gathered buffer, or a list of per-rank wire buffers (``PeerWire.buffers``: the decoder
    then reads the other ranks' bytes straight from their memory, no collective).  ``batched``
    decodes all shards with one launch, straight into their rows of the output tensors;
    ``outputs`` reuses existing BF16 tensors of the given shapes; ``interleave_from`` orders the
    launch's jobs round-robin over the source ranks starting at that rank; ``stage_remote_for``
    (this rank's number, with peer buffers) makes every CTA copy the side bytes of a shard that
    another rank owns into local scratch with full-width requests before it decodes them."""
    from .codec.decode import operand_of
    from .compression.huffman_tables import get_distribution_tables
    from .kernels import dispatch
    from .operations import decompress

    wires = _wires_of(plan, gathered)
    device = wires[0].device
    # A prepared launch pins the wire buffers and the outputs it was made for.  Outputs made
    # here are new on every call, so such a launch could never be reused and is not kept.
    reusable = outputs is not None
    if outputs is None:
        outputs = [torch.empty(shape, dtype=torch.bfloat16, device=device) for shape in shapes]
    key = ("decode", batched, interleave_from, stage_remote_for,
           tuple(_identity(w) for w in wires), tuple(_identity(t) for t in outputs))
    hit = plan.recall(key) if reusable else None
    if hit is not None:
        hit.run()
        return outputs
    views = _views_with_rank(plan, wires)
    if interleave_from is not None:
        views = _interleaved(plan, views, interleave_from % plan.world)
    stage, stage_at = None, 0
    if stage_remote_for is not None and batched:
        remote_bytes = sum(c.size for rank, _, c in views if rank != stage_remote_for)
        stage = torch.empty(max(remote_bytes, 16), dtype=torch.uint8, device=device)
    jobs, direct = [], True
    for rank, shard, compressed in views:
        target = outputs[shard.index]
        rows = target.reshape(()) if target.dim() == 0 else target[shard.row_start:shard.row_stop]
        flat = rows.view(-1).view(torch.int16) if rows.dim() else rows.reshape(1).view(torch.int16)
        if batched and flat.numel() and flat.data_ptr() % 16 == 0:
            job = (operand_of(compressed), flat, compressed.size, flat.numel())
            if stage is not None and rank != stage_remote_for:
                job += (stage[stage_at:stage_at + compressed.size],)   # sizes are block multiples
                stage_at += compressed.size
            jobs.append(job)
        elif flat.numel():
            direct = False
            rows.copy_(decompress(compressed).reshape(rows.shape))
    if jobs:
        block_symbols, lanes, steps, fixed_words = geometry(plan.distribution)
        _, _, rare_length = get_distribution_tables(plan.distribution, device)
        batch = dispatch.decode_batch(jobs, block_symbols=block_symbols, lanes=lanes, steps=steps,
                                      fixed_words=fixed_words, rare_length=rare_length)
        if direct and reusable:
            plan.remember(key, batch)
    return outputs


class PeerWire:
    """Every rank's wire buffer, addressable from this rank's kernels.

    The alternative to ``all_gather_wire``: the buffers live in symmetric memory (one
    allocation per rank, mapped into every peer over NVLink), each rank encodes into its own,
    and ``decode_all(plan, peer.buffers, ..., interleave_from=rank + 1)`` decodes every shard
    by plain loads from the owner's memory - the transfer is the decoder's own input stream, so
    it overlaps the decoding instead of preceding it, and no gathered copy exists.  Measured on
    B200s: faster than all-gather + decode between two GPUs (0.28 ms against 0.38 ms for a
    124 M-parameter set); across eight 0.56 ms against 0.43 ms as it is (the decoder's 32-byte
    side-byte requests use NVLink at half the rate of NCCL's bulk copies) and 0.40 ms with
    ``stage_remote_for=rank``, which is the form to use from four ranks on.  ``fence()``
    orders the ranks on their streams (a one-element all-reduce): call it after encoding and
    before decoding, and again before the buffers are written the next time.

    Loads only: nothing here uses multicast (the multicast binding of the symmetric memory is
    switched off where the installed PyTorch honours ``TORCH_SYMM_MEM_DISABLE_MULTICAST``)."""

    def __init__(self, plan: Plan, rank: int, group=None, device: torch.device | None = None):
        import os

        self.plan, self.rank = plan, rank
        device = (torch.device(device) if device is not None
                  else torch.device("cuda", torch.cuda.current_device()))
        if plan.world == 1:
            self.handle = None
            self.local = torch.zeros(plan.wire_bytes, dtype=torch.uint8, device=device)
            self.buffers = [self.local]
            self.multicast = False
            return
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        if dist.get_world_size(self.group) != plan.world:
            raise ValueError("plan was made for a different number of ranks")
        self.local = symmetric.empty(plan.wire_bytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symmetric.rendezvous(self.local, self.group)
        self.buffers = [self.local if r == rank
                        else self.handle.get_buffer(r, (plan.wire_bytes,), torch.uint8)
                        for r in range(plan.world)]
        self.multicast = bool(getattr(self.handle, "multicast_ptr", 0))
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def fence(self, signal: bool = False) -> None:
        """All ranks' earlier work on their current streams is complete before any rank's later
        work starts (stream-ordered; the host is not blocked).  ``signal``: use the symmetric
        memory's own barrier (flags in the peers' signal pads, a few microseconds) instead of a
        one-element all-reduce."""
        if self.plan.world > 1:
            if signal:
                self.handle.barrier(channel=0)
                return
            import torch.distributed as dist

            dist.all_reduce(self._token, group=self.group)


class WeightSetExchange:
    """One rank's prepared, overlapped step of the weight-set path: encode this rank's shards,
    move every rank's compressed bytes, decode the whole set.

    ``all_gather_wire`` + ``decode_all`` run the collective strictly before a decode of
    everything.  Here the two overlap: the wire buffers live in symmetric memory (two of them,
    used alternately), and after one fence this rank copies the other ranks' buffers into its
    own memory ONE SOURCE AT A TIME on a side stream (each rank starting at its right neighbour,
    so that no source serves all readers at once) while the main stream decodes the sources that
    have already arrived - its own shards first, with no transfer at all.  The step then takes
    about ``encode + max(transfer, decode)`` instead of their sum, and because the buffers
    alternate, ONE fence per step is enough: a rank re-uses a buffer two steps later, and it
    cannot pass the fence in between before every rank has finished reading that buffer.

    The encode side (arena reset + four launches) is captured in a CUDA graph per buffer, so a
    step costs the host a handful of calls.  Copies are plain device-to-device copies out of the
    peers' mapped memory and the decoders read local memory only; nothing uses multicast.

    ``tensors``: this rank's view of the dense weight set (every rank holds all of it; it only
    reads the shards it owns).  ``outputs``: where the decoded set goes (made here if ``None``).
    """

    def __init__(self, plan: Plan, rank: int, tensors: list[torch.Tensor],
                 shapes: list[tuple[int, ...]], group=None,
                 outputs: list[torch.Tensor] | None = None, capture_graphs: bool = True,
                 copy_streams: int = 1, signal_fence: bool = False):
        from .codec.decode import operand_of
        from .compression.huffman_tables import get_distribution_tables
        from .kernels import dispatch

        self.plan, self.rank, self.tensors = plan, rank, tensors
        device = tensors[0].device
        self.outputs = outputs if outputs is not None else [
            torch.empty(shape, dtype=torch.bfloat16, device=device) for shape in shapes]
        self.wires = [PeerWire(plan, rank, group, device) for _ in range(2)]
        self.world = plan.world
        # Local copies of the other ranks' buffers (this rank's own shards are decoded in place).
        self.landing = torch.empty(plan.world * plan.wire_bytes, dtype=torch.uint8, device=device)
        # One side stream by default: with every rank reading a different source at any time the
        # sources never serve two readers at once.  Measured on eight B200s, whole step: one
        # stream 0.39-0.41 ms, two 0.44, three 0.48 (copies that overlap compete at the sources);
        # the signal-pad fence instead of the one-element all-reduce: 0.54.
        self.sides = [torch.cuda.Stream(device=device) for _ in range(max(1, copy_streams))]
        self.signal_fence = signal_fence
        self.order = [(rank + k) % plan.world for k in range(1, plan.world)]
        self.arrived = {source: torch.cuda.Event() for source in self.order}
        self.fenced = torch.cuda.Event()
        self.consumed = torch.cuda.Event()
        self.step_index = 0
        block_symbols, lanes, steps, fixed_words = geometry(plan.distribution)
        _, _, rare_length = get_distribution_tables(plan.distribution, device)
        # One prepared decode launch per (buffer, source rank).
        self.decoders = []
        for wire in self.wires:
            per_source = {}
            for source in range(plan.world):
                local = wire.local if source == rank else self.landing[
                    source * plan.wire_bytes:(source + 1) * plan.wire_bytes]
                jobs, moves = [], []
                for shard, compressed in self._views(local, source):
                    target = self.outputs[shard.index]
                    rows = target.reshape(()) if target.dim() == 0 else target[shard.row_start:shard.row_stop]
                    if rows.numel() == 0:
                        continue
                    if rows.is_contiguous() and rows.data_ptr() % 16 == 0:
                        flat = rows.reshape(-1).view(torch.int16)
                    else:
                        # The batched decoder stores 16 bytes at a time: rows that do not start
                        # on such a boundary are decoded next to the set and copied in.
                        flat = torch.empty(rows.numel(), dtype=torch.int16, device=device)
                        moves.append((rows, flat.view(torch.bfloat16).view(rows.shape)))
                    jobs.append((operand_of(compressed), flat, compressed.size, flat.numel()))
                batch = dispatch.DecodeBatch(
                    jobs, block_symbols=block_symbols, lanes=lanes, steps=steps,
                    fixed_words=fixed_words, rare_length=rare_length) if jobs else None
                per_source[source] = (batch, moves)
            self.decoders.append(per_source)
        # Encode launches, prepared (and captured) per buffer.
        self.encoders = []
        for wire in self.wires:
            encode_rank(plan, rank, tensors, wire=wire.local)          # prepares the launch
            graph = None
            if capture_graphs:
                torch.cuda.synchronize(device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    encode_rank(plan, rank, tensors, wire=wire.local)
            self.encoders.append(graph)
        torch.cuda.synchronize(device)

    def _views(self, wire: torch.Tensor, source: int):
        from .tensor_buffer import TensorBuffer

        plan = self.plan
        start = plan.arena_offset[source] + TensorBuffer.storage_bytes(0, plan.max_free_regions)
        payload = wire[start:start + plan.arena_capacity]
        return [(shard, _compressed_view(plan, wire, shard, slots, payload))
                for shard, slots in zip(plan.shards[source], plan.offsets[source])]

    def encode(self) -> None:
        """This rank's shards into the buffer of the coming step (current stream)."""
        which = self.step_index & 1
        if self.encoders[which] is not None:
            self.encoders[which].replay()
        else:
            encode_rank(self.plan, self.rank, self.tensors, wire=self.wires[which].local)

    def exchange_and_decode(self) -> list[torch.Tensor]:
        """Fence, then copy and decode source by source (see the class text).  Returns the
        decoded weight set (``self.outputs``); stream-ordered on the current stream."""
        which = self.step_index & 1
        wire, decoders = self.wires[which], self.decoders[which]
        main = torch.cuda.current_stream()
        wire.fence(self.signal_fence)              # every rank's buffer of this step is complete
        self.fenced.record(main)
        for side in self.sides:
            side.wait_event(self.fenced)
            side.wait_event(self.consumed)         # the previous step's decoders are done with `landing`
        for k, source in enumerate(self.order):
            side = self.sides[k % len(self.sides)]
            with torch.cuda.stream(side):
                at = source * self.plan.wire_bytes
                self.landing[at:at + self.plan.wire_bytes].copy_(wire.buffers[source], non_blocking=True)
                self.arrived[source].record(side)
        self._decode(decoders[self.rank])
        for source in self.order:
            main.wait_event(self.arrived[source])
            self._decode(decoders[source])
        self.consumed.record(main)
        self.step_index += 1
        return self.outputs

    @staticmethod
    def _decode(prepared) -> None:
        batch, moves = prepared
        if batch is not None:
            batch.run()
        for rows, decoded in moves:
            rows.copy_(decoded)

    def step(self) -> list[torch.Tensor]:
        self.encode()
        return self.exchange_and_decode()


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
