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
