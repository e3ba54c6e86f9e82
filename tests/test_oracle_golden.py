"""Pins the CPU oracle to the reference: every fixture in tests/golden/codec.json was
produced by running the reference's own kernels (tests/golden/make_golden.py)."""
import numpy as np
import pytest

from conftest import sha
from helpers import dist_of, input_of, oracle_compress, region, tables_of
from synth import synth_exact_scale


def _matches(recorded, array) -> bool:
    if isinstance(recorded, dict):
        return recorded["sha"] == sha(array) and recorded["len"] == array.size
    return list(recorded) == np.asarray(array).reshape(-1).tolist()


def _check_components(oracle, c, want, arena=None):
    assert c["center"] == want["center"]
    assert (c["count"], c["tail_bytes"]) == (want["count"], want["tail_bytes"])
    assert list(c["geometry"]) == want["geometry"] and c["size"] == want["size"]
    assert c["encoded"].size == want["encoded_len"]
    assert sha(c["encoded"]) == want["encoded_sha"]
    assert sha(c["side"]) == want["side_sha"]
    assert sha(c["shifted_decode"]) == want["decode_table_sha"]
    assert _matches(want["blocks"], c["blocks"])
    assert oracle.memory_size(c) == want["memory_size"]
    if c["count"] and (arena is None or c["descriptor"][2] == 0):
        for what in ("lanes", "starts", "tail"):
            assert _matches(want[what], region(c, what)), what
    if arena is not None:
        assert c["descriptor"].tolist() == want["descriptor"]
        assert [list(r) for r in oracle.free_regions(arena)] == want["free_regions"]


@pytest.fixture
def linear_lanes(oracle):
    """The reference's other lane mapping (config.lane_mapping = "linear") for one test."""
    oracle.set_lane_mapping("linear")
    yield
    oracle.set_lane_mapping("swizzle")


def _check_codec_cases(oracle, cases):
    for case in cases:
        bits = input_of(case)
        assert sha(bits) == case["input_sha"], "synthetic input generator changed"
        arena = None
        if "buffer" in case:
            arena = oracle.new_arena(case["buffer"])
            oracle.buf_reset(arena)   # the fixture run resets the arena before each of its
            oracle.buf_reset(arena)   # two encodes: generation 3
        c = oracle_compress(oracle, bits, dist_of(case), arena)
        _check_components(oracle, c, case, arena)
        # Words/bytes the reference really writes == what the oracle marks as defined.
        assert int(c["defined"].sum()) == case["word_mask_count"], case["name"]
        assert sha(np.packbits(c["defined"].astype(bool))) == case["word_mask_sha"], case["name"]
        assert int(c["side_defined"].sum()) == case["side_mask_count"], case["name"]
        decoded = oracle.decompress(c)
        assert np.array_equal(decoded, bits) and sha(decoded) == case["decoded_sha"], case["name"]
        if arena is not None:
            assert oracle.buf_free(arena, c["descriptor"]) == 0
            assert [list(r) for r in oracle.free_regions(arena)] == case["free_regions_after_free"]


def test_codec_cases(oracle, golden):
    assert len(golden["codec"]) >= 15
    _check_codec_cases(oracle, golden["codec"])


def test_codec_cases_linear_lane_mapping(oracle, golden, linear_lanes):
    assert len(golden["codec_linear"]) >= 7
    swizzled = {c["name"]: c for c in golden["codec"]}
    for case in golden["codec_linear"]:   # the mapping really changes the payload (rows 0, 1: mask 0)
        if case["n"] > 512:
            assert case["encoded_sha"] != swizzled[case["name"]]["encoded_sha"], case["name"]
    _check_codec_cases(oracle, golden["codec_linear"])


def test_config1_known_answer(oracle, golden):
    torch = pytest.importorskip("torch")
    want = golden["config1"]
    torch.manual_seed(0)
    x = torch.randn(1024, 1024).to(torch.bfloat16)
    bits = x.view(torch.int16).numpy().reshape(-1)
    if sha(bits) != want["input_sha"]:
        pytest.skip("this torch build draws a different randn stream than the fixture's")
    c = oracle_compress(oracle, bits, dist_of(want))
    _check_components(oracle, c, want)
    assert want["memory_size"] == 1446330 and want["center"] == -1 and want["count"] == 4
    assert int(c["defined"].sum()) == want["word_mask_count"]
    assert np.array_equal(oracle.decompress(c), bits)


def test_fused_operation_cases(oracle, golden):
    _check_fused_cases(oracle, golden["pointwise"])


def test_fused_operation_cases_linear_lane_mapping(oracle, golden, linear_lanes):
    assert len(golden["pointwise_linear"]) >= 3
    _check_fused_cases(oracle, golden["pointwise_linear"])


def _check_fused_cases(oracle, cases):
    for case in cases:
        bits = input_of(case)
        assert sha(bits) == case["input_sha"]
        dist = dist_of(case)
        arena = oracle.new_arena(case["buffer"]) if "buffer" in case else None
        a = oracle_compress(oracle, bits, dist, arena)
        n = case["n"]
        if case["op"] == "dual":
            zero = oracle_compress(oracle, np.zeros(n, np.int16), dist, arena)
            dense = oracle.dual(a, zero, case["alpha"])
            side, exps = oracle.dual(a, zero, case["alpha"], dense=False)
        else:
            if case["op"] == "two_scale":
                other = synth_exact_scale(n, case["seed"] + 100)
                assert sha(other) == case["other_sha"]
                kwargs = dict(alpha=case["alpha"], beta=case["beta"], alpha_is_one=False,
                              beta_is_one=False)
            else:
                other = np.zeros(n, np.int16)
                kwargs = dict(alpha=case["alpha"], alpha_is_one=False, beta_is_one=True)
            dense = oracle.pointwise(a, other, oracle.OP_SCALED, **kwargs)
            side, exps = oracle.pointwise(a, other, oracle.OP_SCALED, dense=False, **kwargs)
        assert sha(dense) == case["dense_sha"], case["name"]
        encode, decode, rare = tables_of(dist)
        result = oracle.compress(exps[:n], encode, decode, rare, a["geometry"], precomputed=True,
                                 side=side, arena=arena)
        _check_components(oracle, result, case["result"], arena)
        assert np.array_equal(oracle.decompress(result).view(np.uint16), dense)


def test_allocator_trace(oracle, golden):
    trace = golden["allocator"]
    arena = oracle.new_arena(trace["capacity"], trace["max_free_regions"])
    live = {}
    for step, entry in enumerate(trace["trace"]):
        if entry["op"] == "alloc":
            live[step] = oracle.buf_alloc(arena, entry["arg"])
            assert live[step].tolist() == entry["descriptor"], step
        elif entry["op"] == "free":
            assert oracle.buf_free(arena, live[entry["arg"]]) == entry["status"], step
            assert live[entry["arg"]].tolist() == entry["descriptor"], step
        else:
            oracle.buf_reset(arena)
        assert [list(r) for r in oracle.free_regions(arena)] == entry["free_regions"], step
    statuses = {e.get("status") for e in trace["trace"] if e["op"] == "free"}
    assert {0, 3, 4} <= statuses  # ok, list full, stale/double free all exercised


def test_float_rounding_helpers(oracle):
    """The oracle's BF16 arithmetic against NumPy float32 on values where both are exact."""
    rng = np.random.default_rng(0)
    a = (rng.integers(0, 1 << 16, 4096).astype(np.uint16))
    a = a[(a & 0x7F80) != 0x7F80][:2048]                      # finite
    dist = dist_of(dict(family="GAUSSIAN"))
    c = oracle_compress(oracle, a.view(np.int16), dist)
    as_float = (a.astype(np.uint32) << 16).view(np.float32)
    # x + x and x * 2 are exact in BF16 unless they overflow.
    other = a.copy()
    got = oracle.pointwise(c, other, oracle.OP_ADD)
    want = as_float * np.float32(2)
    want_bits = (want.view(np.uint32) >> 16).astype(np.uint16)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite], want_bits[finite])
    assert np.array_equal(got[~finite] & 0x7FFF, np.full((~finite).sum(), 0x7F80, np.uint16))


def test_optimizer_operations_known_answers(oracle):
    """LERP and EMA_SQUARE of the oracle (PyTorch's float32 formulas, pinned against torch itself
    on the GPU in tests/test_gpu_momentum.py) on values whose results are exact or known: both
    branches of the lerp formula, its end points, and the two roundings of the squared average."""
    def bf16(*values):
        f = np.asarray(values, np.float32)
        return (f.view(np.uint32) >> 16).astype(np.uint16)

    def floats(bits):
        return (np.asarray(bits, np.uint32) << 16).view(np.float32)

    start, end = bf16(1.0, -2.0, 0.5, 3.0, 0.0), bf16(3.0, 6.0, 0.5, -1.0, 8.0)
    assert np.array_equal(floats(oracle.lerp_dense(start, end, 0.25)), [1.5, 0.0, 0.5, 2.0, 2.0])   # w < 0.5
    assert np.array_equal(floats(oracle.lerp_dense(start, end, 0.75)), [2.5, 4.0, 0.5, 0.0, 6.0])   # w >= 0.5
    assert np.array_equal(oracle.lerp_dense(start, end, 0.0), start)
    assert np.array_equal(oracle.lerp_dense(start, end, 1.0), end)          # exact only on the second branch
    # 1 + 2^-9 is not a BF16 value: round to nearest even, from either branch
    assert np.array_equal(floats(oracle.lerp_dense(bf16(1.0), bf16(1.0 + 2.0 ** -7), 0.25)), [1.0])
    assert np.array_equal(floats(oracle.lerp_dense(bf16(1.0), bf16(1.0 + 2.0 ** -7), 0.75)), [1.0078125])
    # the same two operations on a compressed operand
    dist = dist_of(dict(family="GAUSSIAN"))
    values = np.tile(bf16(1.0, -2.0, 0.5, 3.0), 64)
    c = oracle_compress(oracle, values.view(np.int16), dist)
    other = np.tile(bf16(3.0, 6.0, 0.5, -1.0), 64)
    got = oracle.pointwise(c, other, oracle.OP_LERP, 0.25, alpha_is_one=False)
    assert np.array_equal(floats(got[:4]), [1.5, 0.0, 0.5, 2.0])
    got = oracle.pointwise(c, other, oracle.OP_EMA_SQUARE, 0.5, 0.25, alpha_is_one=False, beta_is_one=False)
    assert np.array_equal(floats(got[:4]), [0.5 + 2.25, -1.0 + 9.0, 0.25 + 0.0625, 1.5 + 0.25])
