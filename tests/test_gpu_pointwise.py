"""GPU parity of the fused operations on compressed tensors against the CPU oracle
(float32 fma + round-to-nearest-even, single-rounded BF16 add/multiply) and against PyTorch."""
import numpy as np
import pytest
import torch

from helpers import oracle_compress, tables_of
from gpu_helpers import assert_same_components, bits_of, compress_both, to_dev
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.comp_tensor import CompressedTensor
from losslessly_compressed_tensors_b200.operations import (
    A_compB, A_compBT, a_compA_add_B, a_compA_add_b_B, a_compA_add_compB, compA_add_B,
    compA_mul_B, compress, decompress,
)
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer
from synth import synth_bf16

pytestmark = pytest.mark.gpu

GAUSS = Distribution(DistType.GAUSSIAN)
MEDIUM = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)


def _scalar(v):
    return torch.tensor([v], dtype=torch.float32, device="cuda")


def _recompress(oracle, dist, a_want, side, exps, arena):
    encode, decode, rare = tables_of(dist)
    n = a_want["logical_numel"]
    return oracle.compress(exps[:n], encode, decode, rare, a_want["geometry"], precomputed=True,
                           side=side, arena=arena)


OPS = [
    ("add", dict(op="add")),
    ("mul", dict(op="mul")),
    ("a*A+B", dict(op="scaled", alpha=0.95)),
    ("A+B(alpha_is_one)", dict(op="scaled", alpha=123.0, alpha_is_one=True)),
    ("a*A+b*B", dict(op="scaled", alpha=-0.5, beta=0.3)),
    ("A+b*B", dict(op="scaled", alpha=7.0, beta=-0.02, alpha_is_one=True)),
]
INPUTS = [
    ("normal_ragged", 40000, "normal", GAUSS),
    ("wide_overflow", 32768 + 4321, "wide", GAUSS),
    ("medium_small", 2 * 32768, "normal", MEDIUM),
    ("laplace_big_blocks", 65536 + 99, "outliers", Distribution(DistType.LAPLACE)),
]


def _run_op(a, other, spec, **kwargs):
    if spec["op"] == "add":
        return compA_add_B(a, other, **kwargs)
    if spec["op"] == "mul":
        return compA_mul_B(a, other, **kwargs)
    flag = spec.get("alpha_is_one", False)
    if "beta" in spec:
        return a_compA_add_b_B(a, _scalar(spec["alpha"]), other, _scalar(spec["beta"]),
                               alpha_is_one=flag, **kwargs)
    return a_compA_add_B(a, _scalar(spec["alpha"]), other, alpha_is_one=flag, **kwargs)


def _oracle_op(oracle, a_want, other_bits, spec, dense):
    if spec["op"] == "add":
        return oracle.pointwise(a_want, other_bits, oracle.OP_ADD, dense=dense)
    if spec["op"] == "mul":
        return oracle.pointwise(a_want, other_bits, oracle.OP_MULTIPLY, dense=dense)
    return oracle.pointwise(
        a_want, other_bits, oracle.OP_SCALED, spec["alpha"], spec.get("beta", 1.0),
        alpha_is_one=spec.get("alpha_is_one", False), beta_is_one="beta" not in spec, dense=dense)


@pytest.mark.parametrize("opname,spec", OPS, ids=[o[0] for o in OPS])
@pytest.mark.parametrize("name,n,kind,dist", INPUTS, ids=[i[0] for i in INPUTS])
@pytest.mark.parametrize("buffered", [False, True], ids=["private", "arena"])
@pytest.mark.parametrize("fused", [True, False], ids=["fused", "two-stage"])
def test_compressed_dense_ops(oracle, monkeypatch, opname, spec, name, n, kind, dist, buffered, fused):
    from losslessly_compressed_tensors_b200.codec import pointwise as pointwise_module

    monkeypatch.setattr(pointwise_module, "FUSED_UPDATE", fused)
    bits = synth_bf16(n, 31, kind, -3 if kind == "outliers" else 0)
    other_bits = synth_bf16(n, 32, "normal", -1)
    buffer = TensorBuffer(4 << 20) if buffered else None
    arena = oracle.new_arena(4 << 20) if buffered else None
    x, a, a_want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena)
    other = to_dev(other_bits)

    dense = _run_op(a, other, spec)
    want_dense = _oracle_op(oracle, a_want, other_bits, spec, True)
    assert dense.dtype == torch.bfloat16 and dense.shape == x.shape
    assert np.array_equal(bits_of(dense).view(np.uint16), want_dense)

    comp = _run_op(a, other, spec, dense_output=False, buffer=buffer)
    assert isinstance(comp, CompressedTensor)
    side, exps = _oracle_op(oracle, a_want, other_bits, spec, False)
    want = _recompress(oracle, dist, a_want, side, exps, arena)
    assert_same_components(comp, want, f"{opname}/{name}")
    assert np.array_equal(bits_of(decompress(comp)).view(np.uint16), want_dense)
    if buffered:
        a.free()
        comp.free()
        verify_buffer(buffer)


def test_ops_match_pytorch_expressions():
    """The same checks the reference's own benchmark makes (bitwise against eager PyTorch)."""
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(300000, generator=g) * 2).to(torch.bfloat16).cuda()
    b = (torch.randn(300000, generator=g) * 2).to(torch.bfloat16).cuda()
    m = (1 + 0.01 * torch.randn(300000, generator=g)).to(torch.bfloat16).cuda()
    ca = compress(a, Distribution(DistType.GAUSSIAN, param=2.0))

    def same(x, y):
        return torch.equal(x.view(torch.int16), y.view(torch.int16))

    assert same(compA_add_B(ca, b), a + b)
    assert same(compA_mul_B(ca, m), a * m)
    alpha, beta = _scalar(-0.5), _scalar(-0.02)
    assert same(a_compA_add_B(ca, alpha, b), (a.float() * alpha + b.float()).to(torch.bfloat16))
    two = torch.addcmul(b.float() * beta, a.float(), alpha).to(torch.bfloat16)
    assert same(a_compA_add_b_B(ca, alpha, b, beta), two)
    assert same(decompress(compA_add_B(ca, b, dense_output=False)), a + b)
    cb = compress(b, Distribution(DistType.GAUSSIAN, param=2.0))
    assert same(a_compA_add_compB(ca, alpha, cb), (a.float() * alpha + b.float()).to(torch.bfloat16))


def test_special_values_through_ops(oracle):
    """NaN, infinities, subnormals and signed zeros on both sides of every operation."""
    specials = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x0080, 0x7F7F, 0xFF7F, 0x7F80,
                         0xFF80, 0x7FC0, 0xFFC1, 0x7F81, 0x3F80, 0xBF80, 0x0100], np.uint16)
    left = np.repeat(specials, specials.size)
    right = np.tile(specials, specials.size)
    reps = 40000 // left.size + 1
    left = np.tile(left, reps)[:40000].view(np.int16)
    right = np.tile(right, reps)[:40000].view(np.int16)
    dist = Distribution(DistType.EMPIRICAL, noise_level=NoiseLevel.HIGH)
    x, a, a_want = compress_both(oracle, left, dist)
    other = to_dev(right)
    for opname, spec in OPS:
        got = bits_of(_run_op(a, other, spec)).view(np.uint16)
        want = _oracle_op(oracle, a_want, right, spec, True)
        assert np.array_equal(got, want), opname


@pytest.mark.parametrize("buffered", [False, True], ids=["private", "arena"])
@pytest.mark.parametrize("n,kind_a,kind_b", [(40000, "normal", "laplace"), (32768 + 999, "wide", "normal"),
                                             (70000, "wide", "wide")])
def test_two_compressed_operands(oracle, buffered, n, kind_a, kind_b):
    dist = GAUSS
    buffer = TensorBuffer(4 << 20) if buffered else None
    arena = oracle.new_arena(4 << 20) if buffered else None
    bits_a, bits_b = synth_bf16(n, 41, kind_a), synth_bf16(n, 42, kind_b, -2)
    xa, a, a_want = compress_both(oracle, bits_a, dist, buffer=buffer, arena=arena)
    xb, b, b_want = compress_both(oracle, bits_b, dist, buffer=buffer, arena=arena)
    alpha = 0.37
    dense = a_compA_add_compB(a, _scalar(alpha), b)
    want_dense = oracle.dual(a_want, b_want, alpha)
    assert np.array_equal(bits_of(dense).view(np.uint16), want_dense)
    comp = a_compA_add_compB(a, _scalar(alpha), b, dense_output=False, buffer=buffer)
    side, exps = oracle.dual(a_want, b_want, alpha, dense=False)
    want = _recompress(oracle, dist, a_want, side, exps, arena)
    assert_same_components(comp, want, "dual")
    assert np.array_equal(bits_of(decompress(comp)).view(np.uint16), want_dense)


def test_mixed_geometry_falls_back_to_decode(oracle):
    n = 50000
    a = compress(to_dev(synth_bf16(n, 51, "normal")), GAUSS)
    b = compress(to_dev(synth_bf16(n, 52, "normal")), Distribution(DistType.EMPIRICAL))
    alpha = _scalar(2.0)
    got = a_compA_add_compB(a, alpha, b)
    want = (decompress(a).float() * 2.0 + decompress(b).float()).to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    with pytest.raises(ValueError):
        compA_add_B(a, torch.zeros(n + 1, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):  # result geometry must match the input's
        compA_add_B(a, torch.zeros(n, dtype=torch.bfloat16, device="cuda"), dense_output=False,
                    distribution=Distribution(DistType.EMPIRICAL))
    with pytest.raises(TypeError):
        a_compA_add_B(a, 2.0, torch.zeros(n, dtype=torch.bfloat16, device="cuda"))


def test_momentum_update_steps(oracle):
    """Configuration-4 pattern: m <- 0.95 m + g on compressed state, 20 steps, through LCTTensor
    with a shared arena; every step's compressed components equal the oracle's."""
    dist = MEDIUM
    n = 512 * 1024
    gen = torch.Generator().manual_seed(10)
    m0 = (torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16)
    buffer = TensorBuffer(1 << 20)
    arena = oracle.new_arena(1 << 20)
    state = LCTTensor(m0.cuda().reshape(512, 1024), buffer, dist)
    want = oracle_compress(oracle, bits_of(m0), dist, arena)
    assert_same_components(state.x, want, "init")
    alpha = _scalar(0.95)
    for step in range(20):
        g = (torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16)
        state.mul_add_(alpha, g.cuda().reshape(512, 1024))
        side, exps = oracle.pointwise(want, bits_of(g), oracle.OP_SCALED, 0.95,
                                      alpha_is_one=False, beta_is_one=True, dense=False)
        new = _recompress(oracle, dist, want, side, exps, arena)
        assert oracle.buf_free(arena, want["descriptor"]) in (0, 4)
        want = new
        assert_same_components(state.x, want, f"step {step}")
    dense = state.decompress_free()
    assert np.array_equal(bits_of(dense), oracle.decompress(want))
    verify_buffer(buffer)


def test_lcttensor_wrapper_surface():
    x = (torch.randn(64, 96) * 0.02).to(torch.bfloat16).cuda()
    t = LCTTensor(x, None, Distribution(DistType.EMPIRICAL))
    assert t.shape == x.shape and t.dtype == torch.bfloat16 and t.layout == "LCT compressed"
    assert t.dense_nbytes == x.numel() * 2 and t.nbytes == t.x.memory_size()
    assert torch.equal(t.decompress(), x)
    assert torch.equal(t.t(), x.t())
    y = torch.randn(8, 64, device="cuda").to(torch.bfloat16)
    assert torch.equal(torch.mm(y, t), y @ x)
    t.add_(x)
    assert torch.equal(t.decompress(), x + x)
    other = LCTTensor(x, None, Distribution(DistType.EMPIRICAL))
    t.add_comp_(other, _scalar(-2.0))
    assert torch.equal(t.decompress(), ((x.float() * -2.0) + (x + x).float()).to(torch.bfloat16))
    w = compress(x, Distribution(DistType.EMPIRICAL))
    assert torch.equal(A_compB(y, w), y @ x)
    z = torch.randn(4, 96, device="cuda").to(torch.bfloat16)
    assert torch.equal(A_compBT(z, w), z @ x.T)
    with pytest.raises(ValueError):
        A_compB(z, w)
    t.free()


def test_in_place_updates_recycle_result_storage(oracle):
    """``mul_add_`` / ``add_`` of tensors that share an arena, a codebook and a shape write into
    storage recycled from released values: the number of distinct result storages stays at one
    more than the number of tensors, and every value equals the oracle's at every step."""
    from losslessly_compressed_tensors_b200.codec import pointwise

    pointwise.forget_spare_storage()
    dist = MEDIUM
    shape, n = (96, 1024), 96 * 1024
    gen = torch.Generator().manual_seed(21)
    buffer = TensorBuffer(1 << 20)
    arena = oracle.new_arena(1 << 20)
    starts = [(torch.randn(n, generator=gen) * (1e-3 if i else 30.0)).to(torch.bfloat16)
              for i in range(3)]
    states = [LCTTensor(m.cuda().reshape(shape), buffer, dist) for m in starts]
    wants = [oracle_compress(oracle, bits_of(m), dist, arena) for m in starts]
    alpha, beta = _scalar(0.9), _scalar(-0.5)
    storages = set()
    for step in range(6):
        for i, state in enumerate(states):
            g = (torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16)
            if step % 3 == 0:
                state.mul_add_(alpha, g.cuda().reshape(shape))
                args = (oracle.OP_SCALED, 0.9), dict(alpha_is_one=False, beta_is_one=True)
            elif step % 3 == 1:
                state.mul_add_(alpha, g.cuda().reshape(shape), beta)
                args = (oracle.OP_SCALED, 0.9, -0.5), dict(alpha_is_one=False, beta_is_one=False)
            else:
                state.add_(g.cuda().reshape(shape))
                args = (oracle.OP_ADD,), {}
            side, exps = oracle.pointwise(wants[i], bits_of(g), *args[0], dense=False, **args[1])
            new = _recompress(oracle, dist, wants[i], side, exps, arena)
            assert oracle.buf_free(arena, wants[i]["descriptor"]) in (0, 4)
            wants[i] = new
            assert_same_components(state.x, new, f"step {step} tensor {i}")
            storages.add(state.x.data.data_ptr())
    assert len(storages) == len(states) + 1
    for state, want in zip(states, wants):
        assert np.array_equal(bits_of(state.decompress_free()), oracle.decompress(want))
    verify_buffer(buffer)
    fresh = LCTTensor(starts[1].cuda().reshape(shape), buffer, dist)
    with pytest.raises(ValueError):
        fresh.mul_add_(alpha, torch.zeros(3, 3, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(TypeError):
        fresh.mul_add_(alpha, torch.zeros(shape, dtype=torch.float32, device="cuda"))
    fresh.free()
    verify_buffer(buffer)
    pointwise.forget_spare_storage()
