"""One rank of the CPU (gloo) test of the sharded wire path.  Launched by test_sharded.py with
RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT set.  The codec itself has no CPU path, so each rank
fills its wire buffer from the oracle's output; what is under test is the plan, the wire layout,
the collective and the reconstruction of every shard from the gathered bytes."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    sys.path.insert(0, path)

from helpers import oracle_compress  # noqa: E402
from losslessly_compressed_tensors_b200 import sharded  # noqa: E402
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType  # noqa: E402
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer  # noqa: E402
from oracle import lct_oracle as oracle  # noqa: E402
from synth import synth_bf16  # noqa: E402

SHAPES = [("big", (300, 256)), ("wide", (64, 1024)), ("bias", (768,)), ("mid", (129, 300)),
          ("scalarish", (1,)), ("tall", (1000, 40))]


def weights():
    out = []
    for i, (_, shape) in enumerate(SHAPES):
        n = int(np.prod(shape))
        kind = "wide" if i % 2 else "normal"
        out.append(synth_bf16(n, 700 + i, kind).reshape(shape))
    return out


def fill_wire(plan, rank, tensors):
    """What encode_rank does on a GPU, with the oracle as the encoder."""
    wire = np.zeros(plan.wire_bytes, np.uint8)
    arena = oracle.new_arena(plan.arena_capacity, plan.max_free_regions)
    for shard, slots in zip(plan.shards[rank], plan.offsets[rank]):
        bits = tensors[shard.index][shard.row_start:shard.row_stop].reshape(-1)
        c = oracle_compress(oracle, bits, plan.distribution, arena)
        parts = {"center": np.array([c["center"]], np.int32), "counts": c["counts"],
                 "descriptor": c["descriptor"], "decode_table": c["shifted_decode"],
                 "blocks": c["blocks"], "encoded": c["encoded"], "side": c["side"]}
        for name, (start, nbytes) in slots.items():
            raw = np.ascontiguousarray(parts[name]).view(np.uint8)
            assert raw.size == nbytes, (name, raw.size, nbytes)
            wire[start:start + nbytes] = raw
    start = plan.arena_offset[rank]
    meta = arena["meta"].view(np.uint8)
    wire[start:start + meta.size] = meta
    payload = start + TensorBuffer.storage_bytes(0, plan.max_free_regions)
    wire[payload:payload + plan.arena_capacity] = arena["data"]
    return torch.from_numpy(wire)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    tensors = weights()
    plan = sharded.make_plan(SHAPES, world, Distribution(DistType.GAUSSIAN),
                             row_shard_elements=40000, arena_fraction=0.5)
    wire = fill_wire(plan, rank, tensors)
    gathered = sharded.all_gather_wire(wire, plan)
    assert gathered.numel() == world * plan.wire_bytes
    seen = [np.zeros(t.shape, bool) for t in tensors]
    for shard, c in sharded.views_of(plan, gathered):
        assert c.shape == shard.shape and c.size % c.stream_geometry[0] == 0
        base = int(c.fallback_descriptor[0])
        count, tail = int(c.fallback_count), int(c.fallback_used)
        as_oracle = dict(
            geometry=c.stream_geometry, logical_numel=c.logical_numel, size=c.size,
            center=int(c.center), rare_length=8, shifted_decode=c.decode_table.numpy(),
            encoded=c.data.numpy(), side=c.sign_mantissa.numpy(), blocks=c.fallback_blocks.numpy(),
            lanes=c.fallback_buffer.numpy(), starts=c.fallback_buffer.numpy(),
            tail=c.fallback_buffer.numpy(), offsets=(base, base + count, base + 2 * count),
            count=count, tail_bytes=tail)
        decoded = oracle.decompress(as_oracle).reshape(shard.shape)
        want = tensors[shard.index][shard.row_start:shard.row_stop]
        assert np.array_equal(decoded, want), shard
        seen[shard.index][shard.row_start:shard.row_stop] = True
    assert all(s.all() for s in seen), "some rows were not covered by any shard"
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
