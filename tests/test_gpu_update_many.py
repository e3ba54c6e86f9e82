"""The many-tensor fused update (lct_update_batch): five launches for a list of compressed
tensors must leave, in every result and in the arena, the bytes that one lct_update per tensor
leaves (which tests/test_gpu_pointwise.py pins to the oracle)."""
import numpy as np
import pytest
import torch

from gpu_helpers import bits_of, host, to_dev
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.operations import (
    a_compA_add_B, a_compA_add_b_B, a_compA_add_b_B_many, compress, decompress)
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer)
from losslessly_compressed_tensors_b200.update_plan import UpdatePlan
from synth import synth_bf16

pytestmark = pytest.mark.gpu

MEDIUM = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
CLEAN = Distribution(DistType.GAUSSIAN)

FIELDS = ("data", "sign_mantissa", "center", "decode_table", "fallback_blocks", "fallback_count",
          "fallback_used", "fallback_descriptor")


def _scalar(v):
    return torch.tensor([v], dtype=torch.float32, device="cuda")


def _same(a, b, what):
    assert a.shape == b.shape and a.size == b.size and a.stream_geometry == b.stream_geometry, what
    for name in FIELDS:
        assert np.array_equal(host(getattr(a, name)), host(getattr(b, name))), (what, name)


def _inputs(sizes, kind, seed):
    return [to_dev(synth_bf16(n, seed + i, kind)) for i, n in enumerate(sizes)]


@pytest.mark.parametrize("dist,kind,sizes", [
    (MEDIUM, "normal", [32768 * 3, 5, 40000, 32768, 70001]),       # ragged, tiny, several blocks
    (CLEAN, "wide", [32768 * 2 + 17, 50000, 300]),                  # overflow tails in the arena
], ids=["medium", "overflowing"])
@pytest.mark.parametrize("with_beta", [False, True], ids=["alpha", "alpha-beta"])
def test_many_equals_one_by_one(dist, kind, sizes, with_beta):
    """Two arenas, the same states in both: one gets one call per tensor, the other one call
    for the list; then a second step on the results (sample values carried over)."""
    arenas = [TensorBuffer(4 << 20), TensorBuffer(4 << 20)]
    states = [[compress(x, dist, arena) for x in _inputs(sizes, kind, 100)] for arena in arenas]
    alpha, beta = _scalar(0.95), _scalar(-0.5)
    for step in range(2):
        updates = _inputs(sizes, kind, 200 + 10 * step)
        if with_beta:
            one = [a_compA_add_b_B(s, alpha, g, beta, dense_output=False, buffer=arenas[0],
                                   distribution=dist) for s, g in zip(states[0], updates)]
        else:
            one = [a_compA_add_B(s, alpha, g, dense_output=False, buffer=arenas[0],
                                 distribution=dist) for s, g in zip(states[0], updates)]
        many = a_compA_add_b_B_many(states[1], alpha, updates, beta if with_beta else None,
                                    buffer=arenas[1], distribution=dist)
        assert len(many) == len(one)
        for i, (a, b) in enumerate(zip(one, many)):
            _same(a, b, f"step {step} tensor {i}")
            assert a.memory_size() == b.memory_size()
            assert torch.equal(decompress(a).view(torch.int16), decompress(b).view(torch.int16))
        assert np.array_equal(host(arenas[0]._storage), host(arenas[1]._storage)), f"arena, step {step}"
        for old in states[0] + states[1]:
            old.free()
        states = [one, many]
    if kind == "wide":
        assert sum(int(c.fallback_count.item()) for c in many) > 0   # the tail path really ran
    for arena in arenas:
        verify_buffer(arena)


def test_lcttensor_mul_add_many_matches_pytorch():
    """m <- 0.5 m + g for a list of momentum tensors through LCTTensor.mul_add_many_, three
    steps, against eager PyTorch (the product with 0.5 is exact, so its two roundings equal the
    kernel's one) and against mul_add_ on each."""
    shapes = [(256, 512), (64,), (300, 301), (1024, 128)]
    gen = torch.Generator().manual_seed(7)
    dense = [(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16).cuda() for s in shapes]
    arena = TensorBuffer(1 << 20)
    many = [LCTTensor(x, arena, MEDIUM) for x in dense]
    single = [LCTTensor(x, arena, MEDIUM) for x in dense]
    alpha = _scalar(0.5)
    for _ in range(3):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16).cuda() for s in shapes]
        LCTTensor.mul_add_many_(many, alpha, grads)
        for t, g in zip(single, grads):
            t.mul_add_(alpha, g)
        dense = [(m.float() * alpha + g.float()).to(torch.bfloat16) for m, g in zip(dense, grads)]
        for m, s, want in zip(many, single, dense):
            assert np.array_equal(bits_of(m.decompress()), bits_of(want))
            assert np.array_equal(bits_of(s.decompress()), bits_of(want))
            assert np.array_equal(host(m.x.data), host(s.x.data))
    for t in many + single:
        t.free()
    verify_buffer(arena)


def test_many_rejects_mixed_lists():
    arena = TensorBuffer(1 << 20)
    x = to_dev(synth_bf16(40000, 1, "normal"))
    a = compress(x, MEDIUM, arena)
    b = compress(x, CLEAN, arena)
    alpha = _scalar(1.5)
    with pytest.raises(ValueError):
        a_compA_add_b_B_many([a, b], alpha, [x, x], buffer=arena)
    with pytest.raises(ValueError):
        a_compA_add_b_B_many([a], alpha, [x, x], buffer=arena)
    with pytest.raises(ValueError):
        a_compA_add_b_B_many([a], alpha, [x[:-1]], buffer=arena)
    with pytest.raises(ValueError):
        a_compA_add_b_B_many([a], alpha, [x], buffer=None)


@pytest.mark.parametrize("dist,kind,sizes", [
    (MEDIUM, "normal", [32768 * 3, 5, 40000, 70001]),
    (CLEAN, "wide", [32768 * 2 + 17, 50000, 300]),                  # overflow tails in the arena
], ids=["medium", "overflowing"])
def test_prepared_plan_equals_the_unprepared_call(dist, kind, sizes):
    """UpdatePlan (storage, job tables and work buffers prepared once, two value sets that
    alternate) against mul_add_many_ on a twin arena: same components, same arena, five steps;
    the updates change address at step 3 (the job table is rebuilt) and stay put otherwise."""
    arenas = [TensorBuffer(4 << 20), TensorBuffer(4 << 20)]
    inputs = _inputs(sizes, kind, 300)
    planned = [LCTTensor(x, arenas[0], dist) for x in inputs]
    plain = [LCTTensor(x, arenas[1], dist) for x in inputs]
    alpha = _scalar(0.95)
    plan = UpdatePlan(planned, alpha)
    updates = _inputs(sizes, kind, 400)
    for step in range(5):
        if step == 3:
            updates = [u.clone() for u in _inputs(sizes, kind, 500)]
        elif step:
            for u, fresh in zip(updates, _inputs(sizes, kind, 400 + step)):
                u.copy_(fresh)
        plan.step(updates)
        LCTTensor.mul_add_many_(plain, alpha, updates, group=None)
        for i, (a, b) in enumerate(zip(planned, plain)):
            _same(a.x, b.x, f"step {step} tensor {i}")
            assert a.nbytes == b.nbytes
            assert np.array_equal(bits_of(a.decompress()), bits_of(b.decompress()))
        assert np.array_equal(host(arenas[0]._storage), host(arenas[1]._storage)), f"arena, step {step}"
    assert len(plan.tables) == 2          # 0 -> 1 and 1 -> 0; the first step's table is not kept
    assert set(host(plan.status).tolist()) <= {0, 4}     # 4: a tensor without tails had no region
    # a tensor replaced behind the plan's back
    planned[0].x, planned[1].x = planned[0].x, planned[0].x
    with pytest.raises(ValueError):
        plan.step(updates)
    with pytest.raises(ValueError):
        plan.step(updates[:-1])
    for t in plain:
        t.free()
    for value in plan.values[1 - plan.which]:
        value.free()
    for arena in arenas:
        verify_buffer(arena)
        assert _free_regions_snapshot(arena) == [(0, 4 << 20)]


def test_prepared_plan_with_beta_matches_pytorch():
    shapes = [(128, 512), (300, 301)]
    gen = torch.Generator().manual_seed(11)
    dense = [(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16).cuda() for s in shapes]
    arena = TensorBuffer(1 << 20)
    states = [LCTTensor(x, arena, MEDIUM) for x in dense]
    alpha, beta = _scalar(0.5), _scalar(2.0)
    plan = UpdatePlan(states, alpha, beta)
    for _ in range(4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16).cuda() for s in shapes]
        plan.step(grads)
        dense = [(m.float() * alpha + g.float() * beta).to(torch.bfloat16) for m, g in zip(dense, grads)]
        for m, want in zip(states, dense):
            assert np.array_equal(bits_of(m.decompress()), bits_of(want))
    with pytest.raises(ValueError):
        UpdatePlan([], alpha)
    with pytest.raises(ValueError):
        UpdatePlan([LCTTensor(dense[0], None, MEDIUM)], alpha)
