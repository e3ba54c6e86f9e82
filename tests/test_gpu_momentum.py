"""Optimizer state updates on the compressed form (GPU): ``lerp_`` and ``ema_square_`` must
give the bits of the PyTorch CUDA kernels the reference's optimizers call
(``LCT/components/sparse_utils.py:88-90,193-194``), the compressed components of the oracle,
and the dense by-products (Nesterov direction, new value) of the same launches."""
import numpy as np
import pytest
import torch

from helpers import tables_of
from gpu_helpers import assert_same_components, bits_of
from helpers import oracle_compress
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.codec.geometry import geometry
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.components.dist_configs import momentum_dist, momentum_first_dist
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer

pytestmark = pytest.mark.gpu


def _scalar(v):
    return torch.tensor([v], dtype=torch.float32, device="cuda")


def _values(shape, seed, heavy):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * 1e-2
    if heavy:      # a wide spread of exponents: overflow lanes, cancellation in the lerp
        x = x * torch.exp(torch.randn(shape, generator=g) * 3)
    return x.to(torch.bfloat16)


def _oracle_step(oracle, want, other_bits, op, dist, arena, *scalars):
    side, exps = oracle.pointwise(want, other_bits, op, *scalars, alpha_is_one=False,
                                  beta_is_one=False, dense=False)
    encode, decode, rare = tables_of(dist)
    new = oracle.compress(exps[:want["logical_numel"]], encode, decode, rare, want["geometry"],
                          precomputed=True, side=side, arena=arena)
    assert oracle.buf_free(arena, want["descriptor"]) in (0, 4)
    return new


@pytest.mark.parametrize("shape", [(96, 1024), (37, 1001)], ids=["whole-blocks", "ragged"])
@pytest.mark.parametrize("heavy", [False, True], ids=["plain", "heavy-tailed"])
@pytest.mark.parametrize("weight", [1 - 0.95, 0.95, 0.5, 1 - 0.8], ids=["w.05", "w.95", "w.5", "w.2"])
def test_lerp_matches_torch_and_the_oracle(oracle, shape, heavy, weight):
    dist = momentum_dist
    buffer, arena = TensorBuffer(1 << 20), oracle.new_arena(1 << 20)
    m, g = _values(shape, 1, heavy), _values(shape, 2, heavy)
    state = LCTTensor(m.cuda(), buffer, dist)
    want = oracle_compress(oracle, bits_of(m), dist, arena)
    expect = m.cuda()
    for step in range(3):
        grad = torch.roll(g, step, 0).contiguous()
        expect.lerp_(grad.cuda(), weight)                       # the reference's arithmetic
        assert state.lerp_(grad.cuda(), _scalar(weight))
        want = _oracle_step(oracle, want, bits_of(grad), oracle.OP_LERP, dist, arena,
                            float(np.float32(weight)))
        assert_same_components(state.x, want, f"step {step}")
        assert np.array_equal(bits_of(state.decompress()), bits_of(expect)), step
    state.free()
    verify_buffer(buffer)


@pytest.mark.parametrize("shape", [(64, 2048), (37, 1001)], ids=["whole-blocks", "ragged"])
@pytest.mark.parametrize("mu", [0.95, 0.3])
def test_nesterov_direction_overwrites_the_gradient_like_the_reference(oracle, shape, mu):
    """momentum.lerp_(grad, 1 - mu); grad.lerp_(momentum, mu) - sparse_utils.py:88-90."""
    dist = momentum_dist
    buffer = TensorBuffer(1 << 20)
    m, g = _values(shape, 3, True), _values(shape, 4, True)
    state = LCTTensor(m.cuda(), buffer, dist)
    momentum, grad = m.cuda(), g.cuda()
    momentum.lerp_(grad, 1 - mu)
    direction = grad.clone().lerp_(momentum, mu)
    mine = g.cuda()
    assert state.lerp_(mine, _scalar(1 - mu), nesterov_out=mine, nesterov_weight=_scalar(mu))
    assert np.array_equal(bits_of(state.decompress()), bits_of(momentum))
    assert np.array_equal(bits_of(mine), bits_of(direction))
    # the oracle's formula is the one torch uses, both branches
    assert np.array_equal(oracle.lerp_dense(bits_of(g), bits_of(momentum), float(np.float32(mu))),
                          bits_of(direction).view(np.uint16))
    # a separate output leaves the gradient alone
    other = torch.empty_like(mine)
    fresh = LCTTensor(m.cuda(), buffer, dist)
    assert fresh.lerp_(grad, _scalar(1 - mu), nesterov_out=other, nesterov_weight=_scalar(mu))
    assert np.array_equal(bits_of(other), bits_of(direction))
    assert np.array_equal(bits_of(grad), bits_of(g))
    state.free(); fresh.free()
    verify_buffer(buffer)


def test_second_moment_and_dense_result(oracle):
    """square_avg.mul_(beta2).addcmul_(grad, grad, value=1 - beta2) - sparse_utils.py:194 -
    and the dense copy of the new value that AdamW's weight update reads."""
    dist = momentum_dist
    buffer, arena = TensorBuffer(1 << 20), oracle.new_arena(1 << 20)
    shape, beta2 = (61, 1030), 0.95
    v0 = _values(shape, 5, True).abs()
    state = LCTTensor(v0.cuda(), buffer, dist)
    want = oracle_compress(oracle, bits_of(v0), dist, arena)
    expect = v0.cuda()
    for step in range(3):
        grad = _values(shape, 6 + step, step == 1)
        expect.mul_(beta2).addcmul_(grad.cuda(), grad.cuda(), value=1 - beta2)
        dense = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
        assert state.ema_square_(grad.cuda(), _scalar(beta2), _scalar(1 - beta2), dense_out=dense)
        want = _oracle_step(oracle, want, bits_of(grad), oracle.OP_EMA_SQUARE, dist, arena,
                            float(np.float32(beta2)), float(np.float32(1 - beta2)))
        assert_same_components(state.x, want, f"step {step}")
        assert np.array_equal(bits_of(dense), bits_of(expect))
        assert np.array_equal(bits_of(state.decompress()), bits_of(expect))
    avg = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    before = state.decompress()
    assert state.lerp_(grad.cuda(), _scalar(0.2), dense_out=avg)
    assert np.array_equal(bits_of(avg), bits_of(before.lerp_(grad.cuda(), 0.2)))
    state.free()
    verify_buffer(buffer)


def test_codebook_change_and_the_cases_left_to_the_caller():
    buffer = TensorBuffer(1 << 20)
    m, g = _values((64, 1024), 7, False), _values((64, 1024), 8, False)
    weight = _scalar(0.05)
    first = LCTTensor(torch.zeros_like(m).cuda(), buffer, momentum_first_dist)
    same_geometry = geometry(momentum_first_dist) == geometry(momentum_dist)
    done = first.lerp_(g.cuda(), weight, distribution=momentum_dist)
    assert done == same_geometry
    if done:
        assert first.x.distribution == momentum_dist
        assert np.array_equal(bits_of(first.decompress()),
                              bits_of(torch.zeros_like(m).cuda().lerp_(g.cuda(), 0.05)))
    first.free()
    private = LCTTensor(m.cuda(), None, momentum_dist)               # no arena: not fused
    assert not private.lerp_(g.cuda(), weight)
    assert np.array_equal(bits_of(private.decompress()), bits_of(m))
    state = LCTTensor(m.cuda(), buffer, momentum_dist)
    with pytest.raises(ValueError):
        state.lerp_(g.cuda(), weight, nesterov_out=g.cuda())          # direction without its weight
    with pytest.raises(ValueError):
        state.lerp_(g.cuda(), weight, dense_out=torch.empty(3, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        state.lerp_(g.cuda()[:, :512], weight)
    state.free()
    verify_buffer(buffer)


def test_prepared_plan_does_the_momentum_step_of_every_parameter_at_once(oracle):
    """UpdatePlan with the lerp operation and the Nesterov by-product: same compressed values,
    same directions and the same arena as one ``lerp_`` per tensor, over several steps (the
    plan's two value sets alternate), starting from momentums in the many-zeros codebook."""
    from losslessly_compressed_tensors_b200.codec import pointwise
    from losslessly_compressed_tensors_b200.kernels import dispatch
    from losslessly_compressed_tensors_b200.tensor_buffer import _free_regions_snapshot
    from losslessly_compressed_tensors_b200.update_plan import UpdatePlan

    mu = 0.95
    shapes = [(96, 1024), (37, 1001), (300, 257)]
    one, many = TensorBuffer(2 << 20), TensorBuffer(2 << 20)
    start = [_values(s, 40 + i, i == 1) for i, s in enumerate(shapes)]
    single = [LCTTensor(m.cuda(), one, momentum_first_dist) for m in start]
    batched = [LCTTensor(m.cuda(), many, momentum_first_dist) for m in start]
    plan = UpdatePlan(batched, _scalar(1 - mu), _scalar(mu), operation=pointwise.LERP,
                      emit=dispatch.EMIT_NESTEROV, distribution=momentum_dist)
    for step in range(4):
        grads = [_values(s, 50 + 10 * step + i, step == 2) for i, s in enumerate(shapes)]
        a, b = [g.cuda() for g in grads], [g.cuda() for g in grads]
        for state, g in zip(single, a):
            assert state.lerp_(g, _scalar(1 - mu), distribution=momentum_dist, nesterov_out=g,
                               nesterov_weight=_scalar(mu))
        plan.step(b, dense_outs=b)
        # (the plan reserves all new regions before it releases the old ones, so the regions
        # sit elsewhere in the arena than after one update per tensor: sizes, not offsets, agree)
        assert (sum(size for _, size in _free_regions_snapshot(one))
                == sum(size for _, size in _free_regions_snapshot(many))), step
        for s1, s2, g1, g2 in zip(single, batched, a, b):
            assert s2.x.distribution == momentum_dist
            for name in ("data", "sign_mantissa", "center", "decode_table", "fallback_blocks",
                         "fallback_count", "fallback_used"):
                assert torch.equal(getattr(s1.x, name), getattr(s2.x, name)), (step, name)
            assert torch.equal(s1.x.fallback_descriptor[1:3], s2.x.fallback_descriptor[1:3])
            assert np.array_equal(bits_of(s1.decompress()), bits_of(s2.decompress())), step
            assert np.array_equal(bits_of(g1), bits_of(g2)), step
    expect = start[0].cuda()
    for step in range(4):
        expect.lerp_(_values(shapes[0], 50 + 10 * step, step == 2).cuda(), 1 - mu)
    assert np.array_equal(bits_of(batched[0].decompress()), bits_of(expect))
    with pytest.raises(ValueError):
        plan.step([g.cuda() for g in grads])                        # by-products missing
    with pytest.raises(ValueError):
        UpdatePlan(batched, _scalar(0.1), operation=pointwise.LERP, emit=dispatch.EMIT_NESTEROV)
    for state in single + batched:
        state.free()
    verify_buffer(one)
    verify_buffer(many)
