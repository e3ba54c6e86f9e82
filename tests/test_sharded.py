"""Host logic of the multi-GPU path: the shard plan and wire layout (pure Python), and the
gather + reconstruction with two gloo ranks on CPU."""
import math
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT
from losslessly_compressed_tensors_b200 import sharded
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType


def test_gpt2_small_weight_set():
    shapes = sharded.gpt2_small_shapes()
    assert len(shapes) == 148
    assert sum(math.prod(s) for _, s in shapes) == 124_475_904
    assert sum(1 for _, s in shapes if math.prod(s) <= 3072) == 98


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("row_shard", [None, 4 << 20])
def test_plan_covers_everything_once_and_balances(world, row_shard):
    shapes = sharded.gpt2_small_shapes()
    dist = Distribution(DistType.EMPIRICAL)
    plan = sharded.make_plan(shapes, world, dist, row_shard_elements=row_shard)
    again = sharded.make_plan(shapes, world, dist, row_shard_elements=row_shard)
    assert plan.shards == again.shards and plan.offsets == again.offsets   # same on every rank
    covered = {}
    for rank_shards in plan.shards:
        for shard in rank_shards:
            covered.setdefault(shard.index, []).append((shard.row_start, shard.row_stop))
    for index, (_, shape) in enumerate(shapes):
        spans = sorted(covered[index])
        assert spans[0][0] == 0 and spans[-1][1] == shape[0]
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    loads = [sum(plan.shard_blocks(s) for s in r) for r in plan.shards]
    if row_shard:
        assert max(loads) <= 1.1 * sum(loads) / world + 1
    # wire slots are aligned, disjoint and inside the buffer
    for rank in range(world):
        spans = sorted(slot for slots in plan.offsets[rank] for slot in slots.values())
        assert all(start % 256 == 0 for start, _ in spans)
        assert all(a[0] + a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        assert not spans or spans[-1][0] + spans[-1][1] <= plan.arena_offset[rank] <= plan.wire_bytes
    assert plan.arena_capacity % 16 == 0


def test_split_rows():
    vector = sharded.split_rows("b", 0, (768,), 100)
    assert [s.shape for s in vector] == [(100,)] * 7 + [(68,)]
    parts = sharded.split_rows("w", 3, (10, 7), 21)
    assert [(s.row_start, s.row_stop) for s in parts] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert parts[-1].shape == (1, 7) and all(p.index == 3 for p in parts)
    assert sharded.split_rows("s", 0, (5,), 100)[0].shape == (5,)
    with pytest.raises(ValueError):
        sharded.make_plan([("x", (4,))], 0, Distribution())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_gather_and_reconstruct(oracle):
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dist_worker.py")],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True))
    outputs = [p.communicate(timeout=240)[0] for p in procs]
    for rank, (p, text) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, text[-2000:]
        assert f"rank {rank} ok" in text
