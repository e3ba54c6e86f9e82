"""GPU side of the sharded weight-set path: ranks are emulated one after the other on one GPU
(the collective itself is covered by the gloo test and by bench.py on several GPUs)."""
import numpy as np
import pytest
import torch

from helpers import oracle_compress
from gpu_helpers import assert_same_components, bits_of
from losslessly_compressed_tensors_b200 import sharded
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType
from losslessly_compressed_tensors_b200.tensor_buffer import verify_buffer

pytestmark = pytest.mark.gpu

SHAPES = [("emb", (2000, 96)), ("w1", (96, 384)), ("b1", (384,)), ("w2", (384, 96)), ("b2", (96,)),
          ("ln", (96,)), ("odd", (77, 1031))]


def _weights():
    g = torch.Generator().manual_seed(5)
    out = []
    for i, (_, shape) in enumerate(SHAPES):
        scale = 30.0 if i == 6 else 0.02
        w = torch.randn(shape, generator=g) * scale
        if i == 6:
            w = w * torch.exp(torch.randn(shape, generator=g) * 4)   # forces overflow tails
        out.append(w.to(torch.bfloat16))
    out[5].fill_(1.0)
    out[4].zero_()
    return out


@pytest.mark.parametrize("batched", [True, False], ids=["batched", "per-shard"])
@pytest.mark.parametrize("world,row_shard", [(1, None), (3, None), (3, 30000), (8, 50000)])
def test_encode_gather_decode_round_trip(oracle, world, row_shard, batched):
    dist = Distribution(DistType.EMPIRICAL)
    host = _weights()
    tensors = [w.cuda() for w in host]
    plan = sharded.make_plan(SHAPES, world, dist, row_shard_elements=row_shard, arena_fraction=0.5)
    wires = []
    for rank in range(world):
        wire, compressed, arena = sharded.encode_rank(plan, rank, tensors, batched=batched)
        assert wire.numel() == plan.wire_bytes and len(compressed) == len(plan.shards[rank])
        verify_buffer(arena)
        # every shard equals the oracle's encoding of that shard, arena offsets included
        model = oracle.new_arena(plan.arena_capacity, plan.max_free_regions)
        for shard, c in zip(plan.shards[rank], compressed):
            bits = bits_of(host[shard.index][shard.row_start:shard.row_stop])
            assert_same_components(c, oracle_compress(oracle, bits, dist, model), shard.name)
        wires.append(wire)
    gathered = torch.cat(wires)          # what all_gather_into_tensor leaves on every rank
    assert torch.equal(sharded.all_gather_wire(wires[0], plan), wires[0]) if world == 1 else True
    restored = sharded.decode_all(plan, gathered, [s for _, s in SHAPES], batched=batched)
    for want, got in zip(host, restored):
        assert got.shape == want.shape
        assert np.array_equal(bits_of(got), bits_of(want))
    shards = sum(len(r) for r in plan.shards)
    assert len(sharded.views_of(plan, gathered)) == shards


def test_batched_and_per_shard_paths_write_the_same_wire():
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 2, dist, row_shard_elements=30000, arena_fraction=0.5)
    for rank in range(2):
        one, _, _ = sharded.encode_rank(plan, rank, tensors, batched=False)
        many, _, _ = sharded.encode_rank(plan, rank, tensors, batched=True)
        assert torch.equal(one, many)


def test_wire_buffer_is_reusable():
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 1, dist, arena_fraction=0.5)
    wire, _, _ = sharded.encode_rank(plan, 0, tensors)
    first = wire.clone()
    wire2, _, _ = sharded.encode_rank(plan, 0, tensors, wire=wire)   # second step of a training loop
    assert wire2 is wire and torch.equal(wire, first)
    assert any(k[0] == "encode" for k in plan.prepared)               # the launch was prepared once
    # new values in the same tensors: the prepared launch must pick them up
    tensors[0].mul_(2.0)
    sharded.encode_rank(plan, 0, tensors, wire=wire)
    gathered = sharded.all_gather_wire(wire, plan)
    outputs = sharded.decode_all(plan, gathered, [s for _, s in SHAPES])
    assert all(torch.equal(a, b) for a, b in zip(outputs, tensors))
    tensors[3].add_(1.0)
    sharded.encode_rank(plan, 0, tensors, wire=wire)
    sharded.all_gather_wire(wire, plan, out=gathered)
    again = sharded.decode_all(plan, gathered, [s for _, s in SHAPES], outputs=outputs)
    assert again is outputs and all(torch.equal(a, b) for a, b in zip(outputs, tensors))
    with pytest.raises(ValueError):
        sharded.encode_rank(plan, 0, tensors, wire=torch.zeros(16, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("world,row_shard,start", [(3, 30000, 1), (8, 50000, 5), (1, None, 0)])
def test_decode_from_per_rank_buffers_matches_the_gathered_path(world, row_shard, start):
    """The peer-memory form: decode_all takes one wire buffer per rank (here ordinary local
    tensors standing in for the peers' memory) and may interleave its jobs over the sources."""
    dist = Distribution(DistType.EMPIRICAL)
    host = _weights()
    tensors = [w.cuda() for w in host]
    plan = sharded.make_plan(SHAPES, world, dist, row_shard_elements=row_shard, arena_fraction=0.5)
    wires = [sharded.encode_rank(plan, rank, tensors)[0].clone() for rank in range(world)]
    shapes = [s for _, s in SHAPES]
    for interleave in (None, start):
        restored = sharded.decode_all(plan, wires, shapes, interleave_from=interleave)
        for want, got in zip(host, restored):
            assert np.array_equal(bits_of(got), bits_of(want))
    # side bytes of the shards that rank `start % world` does not own go through local scratch
    staged = sharded.decode_all(plan, wires, shapes, interleave_from=start,
                                stage_remote_for=start % world)
    for want, got in zip(host, staged):
        assert np.array_equal(bits_of(got), bits_of(want))
    # with caller-owned outputs the launch is prepared once per set of buffers and reused
    sharded.decode_all(plan, wires, shapes, outputs=restored, interleave_from=start)
    before = len(plan.prepared)
    sharded.decode_all(plan, wires, shapes, outputs=restored, interleave_from=start)
    assert len(plan.prepared) == before
    order = sharded._interleaved(plan, sharded.views_of(plan, wires), start % world)
    assert len(order) == sum(len(r) for r in plan.shards)
    assert len({id(c) for _, c in order}) == len(order)
    with pytest.raises(ValueError):
        sharded.decode_all(plan, wires[:-1] if world > 1 else [wires[0][:-1]], shapes)


def test_peer_wire_single_rank_is_a_plain_buffer():
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 1, dist, arena_fraction=0.5)
    peer = sharded.PeerWire(plan, 0)
    sharded.encode_rank(plan, 0, tensors, wire=peer.local)
    peer.fence()
    outputs = sharded.decode_all(plan, peer.buffers, [s for _, s in SHAPES], interleave_from=1)
    assert all(torch.equal(a, b) for a, b in zip(outputs, tensors)) and not peer.multicast


def test_repeated_default_calls_keep_nothing_alive():
    """decode_all / all_gather_wire with their defaults make new outputs on every call; a
    prepared launch would pin them (one dense weight set and one gathered buffer per call)."""
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 1, dist, arena_fraction=0.5)
    wire, _, _ = sharded.encode_rank(plan, 0, tensors)
    shapes = [s for _, s in SHAPES]
    for _ in range(3):
        sharded.decode_all(plan, sharded.all_gather_wire(wire, plan), shapes)
    torch.cuda.synchronize()
    held, entries = torch.cuda.memory_allocated(), len(plan.prepared)
    for _ in range(20):
        outputs = sharded.decode_all(plan, sharded.all_gather_wire(wire, plan), shapes)
        del outputs
    torch.cuda.synchronize()
    assert len(plan.prepared) == entries == 0
    assert torch.cuda.memory_allocated() <= held
    # caller-owned buffers: at most `max_prepared` launches are ever kept
    for k in range(plan.max_prepared + 3):
        outs = [torch.empty(shape, dtype=torch.bfloat16, device="cuda") for shape in shapes]
        sharded.decode_all(plan, sharded.all_gather_wire(wire, plan), shapes, outputs=outs)
    assert len(plan.prepared) <= plan.max_prepared


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
def test_overlapped_exchange_on_one_rank(graphs):
    """WeightSetExchange with a world of one: no transfer, but the prepared encode (captured in
    a CUDA graph or not), the alternating wire buffers and the prepared per-source decode."""
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 1, dist, row_shard_elements=30000, arena_fraction=0.5)
    exchange = sharded.WeightSetExchange(plan, 0, tensors, [s for _, s in SHAPES],
                                         capture_graphs=graphs)
    for step in range(4):
        tensors[0].mul_(1.25)          # new values in the same tensors every step
        restored = exchange.step()
        assert all(torch.equal(a, b) for a, b in zip(restored, tensors)), step
    # the wire bytes equal what the unprepared path writes
    wire, _, _ = sharded.encode_rank(plan, 0, tensors)
    assert torch.equal(wire, exchange.wires[(exchange.step_index - 1) & 1].local)


def test_check_reports_shards_whose_tails_did_not_fit():
    """An arena too small for a rank's overflow tails is recorded per shard on the device;
    ``check`` turns that into an exception, and passes a weight set that fitted."""
    dist = Distribution(DistType.EMPIRICAL)
    tensors = [w.cuda() for w in _weights()]
    plan = sharded.make_plan(SHAPES, 2, dist, arena_fraction=0.5)
    wires = [sharded.encode_rank(plan, rank, tensors)[0] for rank in range(2)]
    sharded.check(plan, wires)
    sharded.check(plan, torch.cat(wires))
    small = sharded.make_plan(SHAPES, 2, dist, arena_fraction=0.5)
    small.arena_capacity = 256                       # far below the "odd" tensor's tails
    sharded._lay_out(small)
    wires = [sharded.encode_rank(small, rank, tensors)[0] for rank in range(2)]
    with pytest.raises(RuntimeError, match=r"odd\[0:77\] status [1-9]"):
        sharded.check(small, wires)
