"""Every BASELINE configuration at its full size, byte for byte against the CPU restatement
(the oracle runs its block loops on all host threads: 64 Mi elements in well under a second)."""
import numpy as np
import pytest
import torch

import bench
from helpers import oracle_compress, tables_of
from gpu_helpers import assert_same_components, bits_of
from losslessly_compressed_tensors_b200 import sharded
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.operations import compress, decompress
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer)

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def all_host_threads(oracle):
    oracle.set_threads(0)
    yield


def test_configuration_2_every_component(oracle):
    """8192 x 8192 Laplace weights with outliers, LAPLACE/CLEAN, shared arena: payload, side
    bytes, overflow lists, tails, descriptor and ``memory_size`` equal the oracle's."""
    host = bench.make_workload(1)
    dist = Distribution(DistType.LAPLACE, param=0.02)
    buffer = TensorBuffer(64 << 20)
    arena = oracle.new_arena(64 << 20)
    got = compress(host.cuda(), dist, buffer)
    want = oracle_compress(oracle, bits_of(host), dist, arena)
    assert_same_components(got, want, "configuration 2")
    assert got.memory_size() == oracle.memory_size(want)
    assert np.array_equal(bits_of(decompress(got)), bits_of(host))
    assert _free_regions_snapshot(buffer) == oracle.free_regions(arena)
    got.free()
    verify_buffer(buffer)


def test_configuration_3_sixteen_live_tensors_in_one_arena(oracle):
    """16 live 16384 x 4096 ReLU activations (SPARSE layout) in ONE 64 MiB arena, two batches with
    ``free()`` in between: every descriptor and the free list after every step equal the
    oracle's first-fit arena."""
    dist = Distribution(DistType.LAPLACE, param=1.0, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)
    hosts = []
    for seed in range(4):
        g = torch.Generator().manual_seed(2 + seed)
        hosts.append(torch.randn(16384, 4096, generator=g).relu_().to(torch.bfloat16))
    devices = [h.cuda() for h in hosts]
    buffer = TensorBuffer(64 << 20)
    arena = oracle.new_arena(64 << 20)
    for batch in range(2):
        live, wants = [], []
        for i in range(16):
            k = (i + batch) % 4
            live.append(compress(devices[k], dist, buffer))
            wants.append(oracle_compress(oracle, bits_of(hosts[k]), dist, arena))
            if i % 5 == 0 or i == 15:      # the full comparison is host-bound: a sample of it
                assert_same_components(live[-1], wants[-1], f"batch {batch} tensor {i}")
            else:
                assert live[-1].fallback_descriptor.cpu().tolist() == wants[-1]["descriptor"].tolist()
            assert _free_regions_snapshot(buffer) == oracle.free_regions(arena), (batch, i)
        for i in (0, 7, 15):
            assert np.array_equal(bits_of(decompress(live[i])), bits_of(hosts[(i + batch) % 4]))
        for c, want in zip(live, wants):
            c.free()
            assert oracle.buf_free(arena, want["descriptor"]) == 0
        assert _free_regions_snapshot(buffer) == oracle.free_regions(arena) == [(0, 64 << 20)]
        verify_buffer(buffer)


def test_configuration_4_twenty_steps(oracle):
    """One 4096 x 4096 momentum tensor, GAUSSIAN/MEDIUM, m <- 0.95 m + g for 20 steps through the
    single-launch fused update: every component after every step equals the oracle's."""
    import reference_runner

    dist = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
    momentum, grads = reference_runner.config4_inputs(4096, 4096, 20)
    buffer = TensorBuffer(64 << 20)
    arena = oracle.new_arena(64 << 20)
    state = LCTTensor(momentum.cuda(), buffer, dist)
    want = oracle_compress(oracle, bits_of(momentum), dist, arena)
    assert_same_components(state.x, want, "initial")
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    encode, decode, rare = tables_of(dist)
    for step, grad in enumerate(grads):
        state.mul_add_(alpha, grad.cuda())
        side, exponents = oracle.pointwise(want, bits_of(grad), oracle.OP_SCALED, 0.95,
                                           alpha_is_one=False, beta_is_one=True, dense=False)
        new = oracle.compress(exponents[:want["logical_numel"]], encode, decode, rare,
                              want["geometry"], precomputed=True, side=side, arena=arena)
        assert oracle.buf_free(arena, want["descriptor"]) in (0, 4)
        want = new
        assert_same_components(state.x, want, f"step {step}")
    assert np.array_equal(bits_of(state.decompress_free()), oracle.decompress(want))
    verify_buffer(buffer)


def test_configuration_5_every_rank_wire(oracle):
    """The GPT-2-small-shaped weight set (148 tensors, 157 row-shards) over eight ranks: every
    shard in every rank's wire buffer equals the oracle's encoding of that shard (arena offsets
    included), and the set decodes bit-exactly from the eight buffers."""
    shapes = sharded.gpt2_small_shapes()
    g = torch.Generator().manual_seed(3)
    hosts = []
    for name, shape in shapes:
        if name.endswith("bias"):
            w = torch.zeros(shape)
        elif "ln_" in name:
            w = torch.ones(shape)
        else:
            w = torch.randn(shape, generator=g) * 0.02
        hosts.append(w.to(torch.bfloat16))
    tensors = [h.cuda() for h in hosts]
    dist = Distribution(DistType.EMPIRICAL)
    world = 8
    plan = sharded.make_plan(shapes, world, dist, row_shard_elements=4 << 20)
    wires = []
    for rank in range(world):
        wire, compressed, arena = sharded.encode_rank(plan, rank, tensors)
        model = oracle.new_arena(plan.arena_capacity, plan.max_free_regions)
        for shard, c in zip(plan.shards[rank], compressed):
            source = hosts[shard.index] if hosts[shard.index].dim() == 0 else \
                hosts[shard.index][shard.row_start:shard.row_stop]
            assert_same_components(c, oracle_compress(oracle, bits_of(source), dist, model),
                                   f"rank {rank} {shard.name}[{shard.row_start}:{shard.row_stop}]")
        verify_buffer(arena)
        wires.append(wire)
    restored = sharded.decode_all(plan, wires, [s for _, s in shapes])
    for want, got in zip(hosts, restored):
        assert np.array_equal(bits_of(got), bits_of(want))


def test_arena_lock_timeout_is_a_status_not_a_hang():
    """The arena lock is taken with a bounded number of polls.  With the lock word preset (as a
    crashed holder would leave it) an allocation and a release give up with status 7 and change
    nothing; ``reset()`` restores service."""
    buffer = TensorBuffer(1 << 20)
    held = buffer.allocate(torch.tensor([4096], dtype=torch.int32, device="cuda"))
    assert held.descriptor.cpu().tolist()[2] == 0
    before = _free_regions_snapshot(buffer)
    buffer._lock.fill_(1)
    refused = buffer.allocate(torch.tensor([256], dtype=torch.int32, device="cuda"))
    assert refused.descriptor.cpu().tolist()[:3] == [-1, 0, 7]
    assert int(buffer.free(held).item()) == 7
    assert held.descriptor.cpu().tolist()[2] == 0            # still the owner of its region
    buffer._lock.zero_()
    assert _free_regions_snapshot(buffer) == before           # nothing moved while locked
    buffer._lock.fill_(1)
    # a whole compress against a locked arena: the tails are dropped, nothing hangs or faults
    x = (torch.randn(70000, generator=torch.Generator().manual_seed(1)) *
         torch.exp(torch.randn(70000, generator=torch.Generator().manual_seed(2)) * 6)).to(torch.bfloat16)
    c = compress(x.cuda(), Distribution(DistType.GAUSSIAN), buffer)
    assert c.fallback_descriptor.cpu().tolist()[2] == 7
    buffer.reset()
    fresh = buffer.allocate(torch.tensor([256], dtype=torch.int32, device="cuda"))
    assert fresh.descriptor.cpu().tolist()[:3] == [0, 256, 0]
    verify_buffer(buffer)
