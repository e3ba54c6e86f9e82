"""The reference's other lane mapping, ``config.lane_mapping = "linear"`` (lane l of every row
holds column l), through the same CUDA kernels: reference fixtures, oracle parity for the codec,
the fused operations and the batched weight-set path.  Bit-exact."""
import numpy as np
import pytest
import torch

from conftest import sha
from helpers import dist_of, input_of
from gpu_helpers import assert_same_components, bits_of, compress_both, host, to_dev
from losslessly_compressed_tensors_b200 import config, sharded
from losslessly_compressed_tensors_b200.codec import pointwise as pointwise_module
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.operations import (
    a_compA_add_B, a_compA_add_compB, compress, decompress,
)
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer,
)
from synth import synth_bf16
from test_gpu_pointwise import OPS, _oracle_op, _recompress, _run_op, _scalar

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def linear_lanes(oracle, monkeypatch):
    monkeypatch.setattr(config, "lane_mapping", "linear")
    oracle.set_lane_mapping("linear")
    yield
    oracle.set_lane_mapping("swizzle")
    monkeypatch.undo()
    # hand the default mapping back to the library before any other test launches
    x = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    assert torch.equal(decompress(compress(x, Distribution(DistType.GAUSSIAN))), x)


def test_reference_fixtures_for_the_linear_mapping(oracle, golden):
    swizzled = {c["name"]: c for c in golden["codec"]}
    for case in golden["codec_linear"]:
        bits = input_of(case)
        buffer = arena = None
        if "buffer" in case:
            buffer = TensorBuffer(case["buffer"])
            buffer.reset()
            buffer.reset()
            arena = oracle.new_arena(case["buffer"])
            oracle.buf_reset(arena)
            oracle.buf_reset(arena)
        x, got, want = compress_both(oracle, bits, dist_of(case), buffer=buffer, arena=arena)
        assert_same_components(got, want, case["name"])
        assert sha(host(got.data)) == case["encoded_sha"], case["name"]
        assert sha(host(got.sign_mantissa)) == case["side_sha"], case["name"]
        assert got.memory_size() == case["memory_size"], case["name"]
        if case["n"] > 512:
            assert case["encoded_sha"] != swizzled[case["name"]]["encoded_sha"]
        assert np.array_equal(bits_of(decompress(got)), bits), case["name"]
        if buffer is not None:
            assert _free_regions_snapshot(buffer) == [tuple(r) for r in case["free_regions"]]
            got.free()
            verify_buffer(buffer)


@pytest.mark.parametrize("n", [1, 257, 32769, 65536, 3 * 65536 + 4097])
@pytest.mark.parametrize("kind,dist", [
    ("wide", Distribution(DistType.GAUSSIAN)),
    ("outliers", Distribution(DistType.LAPLACE, param=0.02)),
    ("sparse", Distribution(DistType.LAPLACE, param=1.0, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)),
])
@pytest.mark.parametrize("buffered", [False, True], ids=["private", "arena"])
def test_codec_matches_oracle(oracle, n, kind, dist, buffered):
    bits = synth_bf16(n, 900 + n % 97, kind, -3 if kind == "outliers" else 0)
    buffer = TensorBuffer(4 << 20) if buffered else None
    arena = oracle.new_arena(4 << 20) if buffered else None
    x, got, want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena)
    assert_same_components(got, want, f"{kind}/{n}")
    assert np.array_equal(bits_of(decompress(got)), bits)


@pytest.mark.parametrize("opname,spec", OPS, ids=[o[0] for o in OPS])
@pytest.mark.parametrize("fused", [True, False], ids=["fused", "two-stage"])
@pytest.mark.parametrize("buffered", [False, True], ids=["private", "arena"])
def test_fused_operations_match_oracle(oracle, monkeypatch, opname, spec, fused, buffered):
    monkeypatch.setattr(pointwise_module, "FUSED_UPDATE", fused)
    n, dist = 32768 + 4321, Distribution(DistType.GAUSSIAN)
    bits, other_bits = synth_bf16(n, 31, "wide"), synth_bf16(n, 32, "normal", -1)
    buffer = TensorBuffer(4 << 20) if buffered else None
    arena = oracle.new_arena(4 << 20) if buffered else None
    x, a, a_want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena)
    other = to_dev(other_bits)
    dense = _run_op(a, other, spec)
    want_dense = _oracle_op(oracle, a_want, other_bits, spec, True)
    assert np.array_equal(bits_of(dense).view(np.uint16), want_dense)
    comp = _run_op(a, other, spec, dense_output=False, buffer=buffer)
    side, exps = _oracle_op(oracle, a_want, other_bits, spec, False)
    assert_same_components(comp, _recompress(oracle, dist, a_want, side, exps, arena), opname)
    assert np.array_equal(bits_of(decompress(comp)).view(np.uint16), want_dense)


def test_two_compressed_operands_match_oracle(oracle):
    n, dist = 70000, Distribution(DistType.GAUSSIAN)
    buffer, arena = TensorBuffer(4 << 20), oracle.new_arena(4 << 20)
    xa, a, a_want = compress_both(oracle, synth_bf16(n, 41, "wide"), dist, buffer=buffer, arena=arena)
    xb, b, b_want = compress_both(oracle, synth_bf16(n, 42, "wide", -2), dist, buffer=buffer, arena=arena)
    dense = a_compA_add_compB(a, _scalar(0.37), b)
    assert np.array_equal(bits_of(dense).view(np.uint16), oracle.dual(a_want, b_want, 0.37))
    comp = a_compA_add_compB(a, _scalar(0.37), b, dense_output=False, buffer=buffer)
    side, exps = oracle.dual(a_want, b_want, 0.37, dense=False)
    assert_same_components(comp, _recompress(oracle, dist, a_want, side, exps, arena), "dual")


def test_batched_weight_set_round_trip():
    shapes = [("emb", (2000, 96)), ("w", (96, 384)), ("b", (384,)), ("odd", (77, 1031))]
    g = torch.Generator().manual_seed(5)
    tensors = [(torch.randn(s, generator=g) * (30.0 if i == 3 else 0.02)).to(torch.bfloat16).cuda()
               for i, (_, s) in enumerate(shapes)]
    plan = sharded.make_plan(shapes, 2, Distribution(DistType.EMPIRICAL), row_shard_elements=30000,
                             arena_fraction=0.5)
    wires = []
    for rank in range(2):
        one = sharded.encode_rank(plan, rank, tensors, batched=False)[0].clone()
        many = sharded.encode_rank(plan, rank, tensors, batched=True)[0].clone()
        assert torch.equal(one, many)
        wires.append(many)
    restored = sharded.decode_all(plan, wires, [s for _, s in shapes])
    assert all(torch.equal(a, b) for a, b in zip(restored, tensors))
