"""The buffered pipelines under CUDA-graph capture: every launch goes to the capturing stream,
nothing synchronises the host, and the arena allocator is device-side, so a captured
compress -> decompress -> free (or a fused update) can be replayed on new data."""
import pytest
import torch

from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType
from losslessly_compressed_tensors_b200.operations import a_compA_add_B, compress, decompress
from losslessly_compressed_tensors_b200.tensor_buffer import (
    TensorBuffer, _free_regions_snapshot, verify_buffer,
)

pytestmark = pytest.mark.gpu


def _values(seed, n=3 * 65536 + 777, scale=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * scale).to(torch.bfloat16).cuda()


def test_compress_decompress_free_replays_on_new_data():
    dist = Distribution(DistType.LAPLACE, param=0.02)
    buffer = TensorBuffer(4 << 20)
    source = _values(1)
    for _ in range(2):                       # tables, kernel attributes and allocator pools warm
        c = compress(source, dist, buffer)
        decompress(c)
        c.free()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        c = compress(source, dist, buffer)
        restored = decompress(c)
        c.free()
    for seed in (2, 3, 4):
        # wide exponents on one replay: overflow tails go through the arena inside the graph
        fresh = _values(seed, scale=0.02 if seed != 3 else 300.0)
        if seed == 3:
            fresh = (fresh.float() * torch.exp2(torch.randint(-30, 30, fresh.shape, device="cuda").float())
                     ).to(torch.bfloat16)
        source.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(restored.view(torch.int16), fresh.view(torch.int16)), seed
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]


def test_fused_update_replays():
    dist = Distribution(DistType.GAUSSIAN)
    buffer = TensorBuffer(4 << 20)
    state, grad = _values(5, scale=1e-3), _values(6, scale=1e-3)
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    a = compress(state, dist, buffer)
    for _ in range(2):
        a_compA_add_B(a, alpha, grad, dense_output=False, buffer=buffer).free()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        updated = a_compA_add_B(a, alpha, grad, dense_output=False, buffer=buffer)
        dense = decompress(updated)
        updated.free()
    for seed in (7, 8):
        grad.copy_(_values(seed, scale=1e-3))
        graph.replay()
        torch.cuda.synchronize()
        want = torch.addcmul(grad.float(), state.float(), alpha).to(torch.bfloat16)
        assert torch.equal(dense.view(torch.int16), want.view(torch.int16)), seed
    a.free()
    verify_buffer(buffer)
