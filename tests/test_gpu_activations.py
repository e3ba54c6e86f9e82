"""Compressed activation cache (GPU): lossless, so gradients must not change by one bit, and
every arena region must be back when the backward pass is over."""
import pytest
import torch

from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.components.activations import (
    ActivationCache, compress_weight, compressed_saved_tensors, dense_weight,
)
from losslessly_compressed_tensors_b200.components.dist_configs import act_relu_dist
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer,
)

pytestmark = pytest.mark.gpu


def _model(seed):
    torch.manual_seed(seed)
    model = torch.nn.Sequential(
        torch.nn.Linear(256, 1024), torch.nn.ReLU(), torch.nn.Linear(1024, 1024), torch.nn.GELU(),
        torch.nn.Linear(1024, 64)).cuda().to(torch.bfloat16)
    return model


def _run(model, x, context):
    for p in model.parameters():
        p.grad = None
    x = x.clone().requires_grad_(True)
    with context:
        loss = model(x).float().square().mean()
    loss.backward()
    return [x.grad.clone()] + [p.grad.clone() for p in model.parameters()], loss.detach()


def test_saved_tensor_hooks_keep_gradients_bit_identical_and_release_the_arena():
    import contextlib
    model = _model(0)
    x = torch.randn(512, 256, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)
                    ).to(torch.bfloat16)
    want, want_loss = _run(model, x, contextlib.nullcontext())
    buffer = TensorBuffer(4 << 20)
    cache = ActivationCache(buffer, min_elements=65536)
    got, got_loss = _run(model, x, compressed_saved_tensors(cache=cache))
    assert cache.stored >= 3          # x (512x256) and the 512x1024 activations
    assert torch.equal(got_loss, want_loss)
    for g, w in zip(got, want):
        assert torch.equal(g.view(torch.int16), w.view(torch.int16))
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]


def test_small_fp32_and_parameter_tensors_are_left_alone():
    cache = ActivationCache(None, min_elements=1000)
    small = torch.zeros(10, dtype=torch.bfloat16, device="cuda")
    single = torch.zeros(4096, dtype=torch.float32, device="cuda")
    parameter = torch.nn.Parameter(torch.zeros(4096, dtype=torch.bfloat16, device="cuda"))
    for t in (small, single, parameter):
        handle = cache.store(t)
        assert not handle.is_compressed and handle.load() is t
    assert cache.stored == 0


def test_explicit_store_load_discard_with_a_sparse_codebook():
    buffer = TensorBuffer(1 << 20)
    cache = ActivationCache(buffer, act_relu_dist, min_elements=1)
    x = torch.randn(300, 700, device="cuda").relu().to(torch.bfloat16)
    handle = cache.store(x, track_sizes=True)
    assert handle.is_compressed and cache.compressed_bytes < cache.dense_bytes
    y = handle.load()
    assert torch.equal(y.view(torch.int16), x.view(torch.int16))
    assert handle.load() is y and not handle.is_compressed   # second load: the kept dense tensor
    other = cache.store(x)
    other.discard()
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 1 << 20)]


def test_compress_weight_replaces_the_parameter():
    layer = torch.nn.Linear(512, 256).cuda().to(torch.bfloat16)
    before = layer.weight.detach().clone()
    compress_weight(layer)
    assert isinstance(layer.weight, LCTTensor) and "weight" not in layer._parameters
    assert torch.equal(dense_weight(layer.weight).view(torch.int16), before.view(torch.int16))
    compress_weight(layer)   # idempotent
    assert dense_weight(before) is before


def test_a_forward_without_backward_gives_its_regions_back():
    """Handles that are dropped unloaded (an evaluation forward inside the context, an exception
    before backward) release their arena regions when they are collected."""
    import gc
    model = _model(2)
    x = torch.randn(512, 256, device="cuda").to(torch.bfloat16).requires_grad_(True)
    buffer = TensorBuffer(4 << 20)
    cache = ActivationCache(buffer, act_relu_dist, min_elements=65536)   # a codebook that overflows
    with compressed_saved_tensors(cache=cache):
        loss = model(x).float().square().mean()
    assert cache.stored >= 3
    del loss
    gc.collect()
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]
    handle = cache.store(torch.randn(300, 700, device="cuda").to(torch.bfloat16))
    assert handle.is_compressed
    del handle
    gc.collect()
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]


def test_many_tensor_calls_match_the_one_tensor_calls(oracle=None):
    """compress_many / decompress_many / free_many: the results and the arena of one call per
    tensor in list order, for mixed shapes (ragged, one-dimensional, empty)."""
    from losslessly_compressed_tensors_b200.operations import (
        compress, compress_many, decompress, decompress_many, free_many)

    gen = torch.Generator(device="cuda").manual_seed(3)
    shapes = [(300, 700), (65536,), (0, 8), (17, 3, 1001), (1,)]
    tensors = [(torch.randn(s, device="cuda", generator=gen) *
                torch.exp(torch.randn(s, device="cuda", generator=gen) * 3)).relu().to(torch.bfloat16)
               for s in shapes]
    one, many = TensorBuffer(1 << 20), TensorBuffer(1 << 20)
    singles = [compress(t, act_relu_dist, one) for t in tensors]
    batch = compress_many(tensors, act_relu_dist, many)
    assert _free_regions_snapshot(one) == _free_regions_snapshot(many)
    for a, b, t in zip(singles, batch, tensors):
        assert b.shape == tuple(t.shape) and a.memory_size() == b.memory_size()
        for name in ("data", "sign_mantissa", "center", "decode_table", "fallback_blocks",
                     "fallback_count", "fallback_used", "fallback_descriptor"):
            assert torch.equal(getattr(a, name), getattr(b, name)), name
    assert torch.equal(one.data, many.data)
    for t, d in zip(tensors, decompress_many(batch)):
        assert d.shape == t.shape and torch.equal(d.view(torch.int16), t.view(torch.int16))
    free_many(batch)
    for c in singles:
        c.free()
    assert _free_regions_snapshot(one) == _free_regions_snapshot(many) == [(0, 1 << 20)]
    private = compress_many(tensors[:2], act_relu_dist, None)       # no arena: one call each
    assert all(torch.equal(decompress(c), t) for c, t in zip(private, tensors))


@pytest.mark.parametrize("batch", [0, 2], ids=["flush-at-exit", "groups-of-two"])
def test_batching_cache_keeps_gradients_bit_identical(batch):
    import contextlib
    import gc
    model = _model(4)
    x = torch.randn(512, 256, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)
                    ).to(torch.bfloat16)
    want, want_loss = _run(model, x, contextlib.nullcontext())
    buffer = TensorBuffer(4 << 20)
    cache = ActivationCache(buffer, min_elements=65536, batch=batch)
    got, got_loss = _run(model, x, compressed_saved_tensors(cache=cache))
    assert cache.stored >= 3 and torch.equal(got_loss, want_loss)
    for g, w in zip(got, want):
        assert torch.equal(g.view(torch.int16), w.view(torch.int16))
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]
    # explicit use: stored tensors stay dense until the flush, and a load before it is free
    a = torch.randn(300, 700, device="cuda").relu().to(torch.bfloat16)
    cache = ActivationCache(buffer, act_relu_dist, min_elements=1, batch=0)
    first, second, third = cache.store(a), cache.store(a * 2), cache.store(a * 3)
    assert not first.is_compressed and first.load() is not None
    cache.flush()
    assert second.is_compressed and third.is_compressed and not first.is_compressed
    storage = {second._compressed.data.data_ptr(), third._compressed.data.data_ptr()}
    assert torch.equal(second.load(), a * 2)            # decodes the whole group ...
    assert not third.is_compressed and torch.equal(third.load(), a * 3)
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]     # ... and releases it
    fourth = cache.store(a * 5)
    cache.flush()
    assert fourth._compressed.data.data_ptr() in storage        # the released storage is reused
    assert torch.equal(fourth.load(), a * 5)
    fourth = cache.store(a)
    cache.flush()
    del fourth
    gc.collect()
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]
    with pytest.raises(ValueError):
        ActivationCache(None, batch=4)
