"""GPU parity: compress / decompress through the public API (-> C ABI -> sm_100a kernels)
against the CPU oracle and the reference-generated fixtures.  Bit-exact everywhere."""
import numpy as np
import pytest
import torch

from conftest import sha
from helpers import dist_of, input_of, oracle_compress
from gpu_helpers import assert_same_components, bits_of, compress_both, host, to_dev
from losslessly_compressed_tensors_b200.comp_format import (
    Distribution, DistType, NoiseLevel, StorageLayout,
)
from losslessly_compressed_tensors_b200.operations import compress, decompress
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer,
)

pytestmark = pytest.mark.gpu


def _cpu_randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def _laplace(n, seed, scale):
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=g) - 0.5
    return -scale * torch.sign(u) * torch.log1p(-2.0 * u.abs())


def test_golden_cases_private_and_buffered(oracle, golden):
    """The reference fixtures: same bytes in every component, same memory_size, same arena state."""
    for case in golden["codec"]:
        bits = input_of(case)
        dist = dist_of(case)
        buffer = arena = None
        if "buffer" in case:
            buffer = TensorBuffer(case["buffer"])
            buffer.reset()
            buffer.reset()  # fixture generation: generation 3
            arena = oracle.new_arena(case["buffer"])
            oracle.buf_reset(arena)
            oracle.buf_reset(arena)
        x, got, want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena)
        assert_same_components(got, want, case["name"])
        assert sha(host(got.data)) == case["encoded_sha"], case["name"]
        assert sha(host(got.sign_mantissa)) == case["side_sha"], case["name"]
        assert got.memory_size() == case["memory_size"], case["name"]
        restored = decompress(got)
        assert restored.shape == x.shape and restored.dtype == torch.bfloat16
        assert np.array_equal(bits_of(restored), bits), case["name"]
        if buffer is not None:
            assert _free_regions_snapshot(buffer) == [tuple(r) for r in case["free_regions"]]
            got.free()
            verify_buffer(buffer)
            assert _free_regions_snapshot(buffer) == [
                tuple(r) for r in case["free_regions_after_free"]]


def test_config1_known_answer(oracle, golden):
    """BASELINE configuration 1: 1024x1024 N(0,1), GAUSSIAN, no buffer."""
    want = golden["config1"]
    torch.manual_seed(0)
    x = torch.randn(1024, 1024).to(torch.bfloat16)
    bits = bits_of(x)
    if sha(bits) != want["input_sha"]:
        pytest.skip("this torch build draws a different randn stream than the fixture's")
    c = compress(x.cuda(), Distribution(DistType.GAUSSIAN))
    assert int(c.center.item()) == -1 and c.memory_size() == 1446330
    assert sha(host(c.data)) == want["encoded_sha"]
    assert sha(host(c.sign_mantissa)) == want["side_sha"]
    assert host(c.fallback_lanes).tolist() == want["lanes"]
    assert host(c.fallback_starts).tolist() == want["starts"]
    assert host(c.fallback_buffer).tolist() == want["tail"]
    assert host(c.fallback_blocks).tolist() == want["blocks"]
    y = decompress(c)
    assert torch.equal(y.cpu().view(torch.int16), x.view(torch.int16))


CASES = [
    # name, values(fp32 CPU tensor factory), Distribution
    ("gauss_2d", lambda: _cpu_randn((1500, 700), 1), Distribution(DistType.GAUSSIAN)),
    ("laplace_outliers", lambda: _laplace(3 * 65536 + 777, 2, 0.02) *
     (1 + 99 * (torch.rand(3 * 65536 + 777, generator=torch.Generator().manual_seed(3)) < 1e-3)),
     Distribution(DistType.LAPLACE, param=0.02)),
    ("relu_sparse", lambda: _cpu_randn((600, 1000), 4).relu(),
     Distribution(DistType.LAPLACE, param=1.0, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)),
    ("momentum_medium", lambda: _cpu_randn((512, 1024), 5, 1e-3),
     Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)),
    ("empirical_weights", lambda: _cpu_randn((768, 2304), 6, 0.02), Distribution(DistType.EMPIRICAL)),
    ("uniform_high", lambda: (torch.rand(200000, generator=torch.Generator().manual_seed(7)) - 0.5) * 64,
     Distribution(DistType.EMPIRICAL, noise_level=NoiseLevel.HIGH)),
    ("gamma", lambda: _cpu_randn((100000,), 8).abs() ** 1.5, Distribution(DistType.GAMMA)),
    ("mismatched_codebook", lambda: _laplace(300000, 9, 1.5), Distribution(DistType.GAUSSIAN)),
    ("huge_range", lambda: _cpu_randn((70000,), 10) * torch.exp(_cpu_randn((70000,), 11, 12.0)),
     Distribution(DistType.GAUSSIAN)),
]


@pytest.mark.parametrize("name,make,dist", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("buffered", [False, True], ids=["private", "arena"])
def test_random_tensors_match_oracle(oracle, name, make, dist, buffered):
    values = make().to(torch.bfloat16)
    bits = bits_of(values)
    buffer = TensorBuffer(8 << 20) if buffered else None
    arena = oracle.new_arena(8 << 20) if buffered else None
    x, got, want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena,
                                 shape=tuple(values.shape))
    assert_same_components(got, want, name)
    assert got.memory_size() == oracle.memory_size(want)
    assert got.shape == tuple(values.shape) and got.layout is StorageLayout.COMPRESSED
    restored = decompress(got)
    assert restored.shape == values.shape
    assert np.array_equal(bits_of(restored), bits)
    if buffered:
        assert _free_regions_snapshot(buffer) == oracle.free_regions(arena)


@pytest.mark.parametrize("n", [1, 2, 255, 256, 257, 511, 32767, 32768, 32769, 65535, 65536, 65537,
                               3 * 32768 + 12345])
@pytest.mark.parametrize("family,level", [(DistType.GAUSSIAN, NoiseLevel.CLEAN),
                                          (DistType.EMPIRICAL, NoiseLevel.CLEAN),
                                          (DistType.LAPLACE, NoiseLevel.SPARSE)])
def test_ragged_sizes(oracle, n, family, level):
    """Every block-boundary neighbourhood, with data wide enough that lanes overflow."""
    from synth import synth_bf16

    bits = synth_bf16(n, 100 + n % 97, "wide" if n % 2 else "laplace")
    dist = Distribution(family, noise_level=level)
    x, got, want = compress_both(oracle, bits, dist)
    assert_same_components(got, want, f"n={n}")
    assert np.array_equal(bits_of(decompress(got)), bits)


def test_empty_tensor():
    x = torch.empty(0, 7, dtype=torch.bfloat16, device="cuda")
    c = compress(x, Distribution(DistType.GAUSSIAN))
    assert c.size == 0 and c.logical_numel == 0
    y = decompress(c)
    assert y.shape == (0, 7) and y.dtype == torch.bfloat16
    buffered = compress(x, Distribution(DistType.GAUSSIAN), TensorBuffer(4096))
    buffered.free()
    assert decompress(buffered).numel() == 0


def test_unaligned_and_strided_sources(oracle):
    """Views that start 2 bytes into an allocation, and non-contiguous inputs."""
    base = _cpu_randn((70001,), 21).to(torch.bfloat16).cuda()
    dist = Distribution(DistType.GAUSSIAN)
    for view in (base[1:], base[3:40000], base[:65536].reshape(256, 256).t()):
        bits = bits_of(view)
        c = compress(view, dist)
        assert_same_components(c, oracle_compress(oracle, bits, dist), "view")
        y = decompress(c)
        assert y.shape == view.shape and torch.equal(y, view)


def test_allow_raw_keeps_small_tensors_dense():
    x = _cpu_randn((768,), 22, 0.02).to(torch.bfloat16).cuda()
    dist = Distribution(DistType.EMPIRICAL)
    raw = compress(x, dist, allow_raw=True)
    assert raw.layout is StorageLayout.RAW and raw.memory_size() == x.numel() * 2
    assert torch.equal(decompress(raw), x)
    packed = compress(x, dist, allow_raw=False)
    assert packed.layout is StorageLayout.COMPRESSED and packed.memory_size() == 95280
    big = _cpu_randn((200000,), 23).to(torch.bfloat16).cuda()
    assert compress(big, dist, allow_raw=True).layout is StorageLayout.COMPRESSED


def test_special_values_round_trip():
    """NaN payloads, infinities, subnormals, signed zeros: every one of the 65536 bit patterns."""
    bits = np.arange(65536, dtype=np.uint16).view(np.int16)
    bits = np.tile(bits, 3)[: 3 * 65536 - 5]
    for dist in (Distribution(DistType.GAUSSIAN), Distribution(DistType.EMPIRICAL),
                 Distribution(DistType.LAPLACE, noise_level=NoiseLevel.HIGH)):
        c = compress(to_dev(bits), dist)
        assert np.array_equal(bits_of(decompress(c)), bits)


def test_non_bf16_input_is_rejected():
    with pytest.raises(TypeError):
        compress(torch.zeros(8, device="cuda"), Distribution())


def test_allocator_trace_on_device(golden):
    """The reference's allocator script through TensorBuffer: same descriptors, statuses, free lists."""
    trace = golden["allocator"]
    buffer = TensorBuffer(trace["capacity"], max_free_regions=trace["max_free_regions"])
    live = {}
    for step, entry in enumerate(trace["trace"]):
        if entry["op"] == "alloc":
            live[step] = buffer.allocate(torch.tensor([entry["arg"]], dtype=torch.int32, device="cuda"))
            assert live[step].descriptor.tolist() == entry["descriptor"], step
        elif entry["op"] == "free":
            status = buffer.free(live[entry["arg"]])
            assert int(status.item()) == entry["status"], step
            assert live[entry["arg"]].descriptor.tolist() == entry["descriptor"], step
        else:
            buffer.reset()
        assert _free_regions_snapshot(buffer) == [tuple(r) for r in entry["free_regions"]], step
        if entry["op"] != "free" or entry["status"] != 3:
            verify_buffer(buffer)


def test_allocator_random_sequences_match_model(oracle):
    rng = np.random.default_rng(5)
    for regions in (4, 256):
        buffer = TensorBuffer(1 << 16, max_free_regions=regions)
        arena = oracle.new_arena(1 << 16, regions)
        live = []
        for _ in range(300):
            if live and rng.random() < 0.45:
                got, want = live.pop(int(rng.integers(len(live))))
                status = buffer.free(got)
                assert int(status.item()) == oracle.buf_free(arena, want)
            else:
                items = int(rng.integers(0, 40))
                nbytes = int(rng.integers(0, 3000))
                got = buffer.allocate_with_items(
                    torch.tensor([nbytes], dtype=torch.int32, device="cuda"),
                    torch.tensor([items], dtype=torch.int32, device="cuda"), 2)
                want = oracle.buf_alloc(arena, nbytes, items, 2)
                assert got.descriptor.tolist() == want.tolist()
                live.append((got, want))
        assert _free_regions_snapshot(buffer) == oracle.free_regions(arena)
    with pytest.raises(ValueError):
        TensorBuffer(1024, max_free_regions=3)
    with pytest.raises(ValueError):
        buffer.free(TensorBuffer(1024).allocate(torch.tensor([16], device="cuda")))


def test_arena_exhaustion_is_reported_not_fatal(oracle):
    """An arena too small for the tails: status 1 in the descriptor, no write outside the arena,
    and the arena stays usable."""
    from synth import synth_bf16

    bits = synth_bf16(2 * 32768, 77, "wide")
    buffer = TensorBuffer(1024)
    guard_before = buffer._storage.clone()
    c = compress(to_dev(bits), Distribution(DistType.GAUSSIAN), buffer)
    assert c.fallback_descriptor.tolist()[:3] == [-1, 0, 1]
    assert int(c.fallback_count.item()) > 0
    regions = buffer.max_free_regions
    assert torch.equal(buffer._storage[8 * regions + 12:], guard_before[8 * regions + 12:])
    from losslessly_compressed_tensors_b200.tensor_buffer import Allocation

    assert int(buffer.free(Allocation(c.fallback_descriptor, buffer)).item()) == 4  # nothing to free
    c.free()
    verify_buffer(buffer)
    small = compress(to_dev(synth_bf16(1000, 78, "normal")), Distribution(DistType.GAUSSIAN), buffer)
    assert np.array_equal(bits_of(decompress(small)), synth_bf16(1000, 78, "normal"))


def test_shared_arena_many_live_tensors(oracle):
    """Configuration-3 pattern at reduced size: live tensors share one arena, free between batches."""
    dist = Distribution(DistType.LAPLACE, param=1.0, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)
    buffer = TensorBuffer(4 << 20)
    arena = oracle.new_arena(4 << 20)
    for batch in range(3):
        live = []
        for i in range(16):
            values = _cpu_randn((128, 1024), 1000 + 16 * batch + i).relu().to(torch.bfloat16)
            bits = bits_of(values)
            x, got, want = compress_both(oracle, bits, dist, buffer=buffer, arena=arena)
            assert_same_components(got, want, f"batch {batch} tensor {i}")
            live.append((bits, got, want))
        for bits, got, want in live:
            assert np.array_equal(bits_of(decompress(got)), bits)
        for order, (bits, got, want) in enumerate(live[::2] + live[1::2]):
            got.free()
            assert oracle.buf_free(arena, want["descriptor"]) == 0
        verify_buffer(buffer)
        assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]


@pytest.mark.parametrize("n,kind", [(1, "normal"), (65537, "normal"), (3 * 65536 + 77, "wide"),
                                    (40 * 65536, "laplace")])
def test_single_call_pipeline_matches_staged_calls(monkeypatch, n, kind):
    """lct_compress (four overlapping launches behind one call) leaves exactly the bytes of the four
    separate calls: every component, the arena contents and the allocator state."""
    from losslessly_compressed_tensors_b200.codec import encode as encode_module
    if kind == "laplace":
        values = _laplace(n, 5, 0.02)
    elif kind == "wide":   # exponents far outside the codebook: many overflowing lanes
        values = _cpu_randn((n,), 6) * torch.exp2(torch.randint(-20, 20, (n,),
                                                                generator=torch.Generator().manual_seed(7)).float())
    else:
        values = _cpu_randn((n,), 8)
    x = values.to(torch.bfloat16).cuda()
    dist = Distribution(DistType.LAPLACE, param=0.02)
    results = []
    for single in (True, False):
        monkeypatch.setattr(encode_module, "SINGLE_CALL_PIPELINE", single)
        buffer = TensorBuffer(8 << 20)
        first = compress(x, dist, buffer)     # two live tensors: the second reservation starts
        second = compress(x, dist, buffer)    # behind the first one
        torch.cuda.synchronize()
        assert torch.equal(decompress(second).view(torch.int16), x.view(torch.int16))
        results.append((first, second, buffer))
    (a1, a2, abuf), (b1, b2, bbuf) = results
    for got, want in ((a1, b1), (a2, b2)):
        for field in ("data", "sign_mantissa", "center", "decode_table", "fallback_blocks",
                      "fallback_count", "fallback_used", "fallback_descriptor"):
            assert torch.equal(getattr(got, field), getattr(want, field)), field
        assert got.memory_size() == want.memory_size()
    assert torch.equal(abuf._storage, bbuf._storage)
    assert _free_regions_snapshot(abuf) == _free_regions_snapshot(bbuf)


def test_full_size_round_trip_properties():
    """BASELINE configuration 2 at full size (64 Mi elements): size-independent properties."""
    n = 8192 * 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    u = torch.rand(n, device="cuda", generator=g) - 0.5
    values = -0.02 * torch.sign(u) * torch.log1p(-2.0 * u.abs())
    outlier = torch.rand(n, device="cuda", generator=g) < 1e-4
    values = torch.where(outlier, values * 100, values).to(torch.bfloat16).reshape(8192, 8192)
    del u, outlier
    dist = Distribution(DistType.LAPLACE, param=0.02)
    buffer = TensorBuffer(64 << 20)
    for buf in (None, buffer):
        c = compress(values, dist, buf)
        assert c.stream_geometry == (65536, 256, 256, 25)
        y = decompress(c)
        assert torch.equal(y.view(torch.int16), values.view(torch.int16))
        ratio = values.numel() * 2 / c.memory_size()
        assert 1.40 < ratio < 1.44, ratio
        again = compress(y, dist, buf)   # encode is a pure function of the values
        assert torch.equal(again.data, c.data) and torch.equal(again.sign_mantissa, c.sign_mantissa)
        assert torch.equal(again.center, c.center)
        assert torch.equal(again.fallback_blocks, c.fallback_blocks)
        c.free()
        again.free()
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 64 << 20)]
