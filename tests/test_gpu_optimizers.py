"""Optimizers with compressed state (GPU).  The codec is lossless, so compressed and dense
state must give bit-identical trajectories wherever both variants run the same arithmetic; the
fully fused SGDM path is checked against the fp32-fma formulas it implements."""
import pytest
import torch

from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.components.dist_configs import weight_dist
from losslessly_compressed_tensors_b200.components.sparse_utils import (
    SparseAdamW, SparseMuon, SparseSGDM,
)
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, verify_buffer, _free_regions_snapshot

pytestmark = pytest.mark.gpu

SHAPES = [(300, 257), (64, 1024), (129, 33)]


def _params(seed, scale=0.02):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(s, generator=g) * scale).to(torch.bfloat16).cuda() for s in SHAPES]


def _grads(seed, step):
    g = torch.Generator().manual_seed(1000 * seed + step)
    return [(torch.randn(s, generator=g) * 1e-2).to(torch.bfloat16).cuda() for s in SHAPES]


def _bits(t):
    return t.view(torch.int16)


def _fma(a, alpha, b):
    """bf16(fma(f32(a), alpha, f32(b))) - the arithmetic of the fused kernels."""
    return torch.addcmul(b.float(), a.float(), alpha).to(torch.bfloat16)


@pytest.mark.parametrize("compressed_params", [False, True], ids=["dense-params", "lct-params"])
def test_sgdm_fused_path_matches_fma_formulas(compressed_params):
    buffer = TensorBuffer(8 << 20)
    dense = _params(1)
    params = [LCTTensor(p.clone(), buffer, weight_dist) if compressed_params else p.clone() for p in dense]
    optimizer = SparseSGDM(params, lr=0.1, momentum=0.9, buffer=buffer, compressed=True)
    momentum = torch.tensor([0.9], dtype=torch.float32, device="cuda")
    neg_lr = torch.tensor([-0.1], dtype=torch.float32, device="cuda")
    want_m = [None] * len(dense)
    for step in range(4):
        grads = _grads(1, step)
        for p, g in zip(params, grads):
            p.grad = g
        optimizer.step()
        for i, g in enumerate(grads):
            want_m[i] = g.clone() if want_m[i] is None else _fma(want_m[i], momentum, g)
            dense[i] = _fma(want_m[i], neg_lr, dense[i])
        for i, p in enumerate(params):
            got = p.decompress() if compressed_params else p
            assert torch.equal(_bits(got), _bits(dense[i])), (step, i)
            assert torch.equal(_bits(optimizer.momentums[i].decompress()), _bits(want_m[i])), (step, i)
    optimizer.zero_grad()
    assert all(p.grad is None for p in params)
    for state in optimizer.momentums:
        state.free()
    for p in params:
        if compressed_params:
            p.free()
    verify_buffer(buffer)
    assert _free_regions_snapshot(buffer) == [(0, 8 << 20)]


@pytest.mark.parametrize("zero_first_step", [False, True])
def test_muon_compressed_state_follows_the_dense_trajectory(zero_first_step):
    buffer = TensorBuffer(8 << 20)
    a, b = _params(2), _params(2)
    with_state = SparseMuon(a, lr=0.02, weight_decay=0.01, buffer=buffer, compressed=True,
                            zero_first_step=zero_first_step, ns_iters=3)
    dense_state = SparseMuon(b, lr=0.02, weight_decay=0.01, compressed=False, ns_iters=3)
    for step in range(3):
        for pa, pb, g in zip(a, b, _grads(2, step)):
            pa.grad, pb.grad = g.clone(), g.clone()
        with_state.step()
        dense_state.step()
        for i, (pa, pb) in enumerate(zip(a, b)):
            assert torch.equal(_bits(pa), _bits(pb)), (step, i)
        for ma, mb in zip(with_state.momentums, dense_state.momentums):
            assert isinstance(ma, LCTTensor)
            assert torch.equal(_bits(ma.decompress()), _bits(mb))
    verify_buffer(buffer)


def test_muon_on_compressed_weights_uses_the_fused_decay_and_update():
    buffer = TensorBuffer(8 << 20)
    dense = _params(3)
    params = [LCTTensor(p.clone(), buffer, weight_dist) for p in dense]
    optimizer = SparseMuon(params, lr=0.02, weight_decay=0.1, buffer=buffer, ns_iters=2)
    shadow = SparseMuon([p.clone() for p in dense], lr=0.02, weight_decay=0.1, compressed=False,
                        ns_iters=2)
    for step in range(2):
        grads = _grads(3, step)
        for p, q, g in zip(params, shadow.params, grads):
            p.grad, q.grad = g.clone(), g.clone()
        # the dense update each parameter will receive (same momentum arithmetic in both)
        before = [p.decompress() for p in params]
        optimizer.step()
        shadow.step()
        for i, p in enumerate(params):
            # recover the update from the shadow's momentum: rerun its arithmetic on copies
            got = p.decompress()
            assert got.shape == before[i].shape and got.dtype == torch.bfloat16
            assert torch.isfinite(got.float()).all()
            # alpha * x + beta * update in fp32 with one rounding: never further than one BF16
            # step of the two-rounding dense formula the shadow applies
            ref = shadow.params[i]
            assert (got.float() - ref.float()).abs().max() <= 2.0 ** -7 * ref.float().abs().max()
        for ma, mb in zip(optimizer.momentums, shadow.momentums):
            assert torch.equal(_bits(ma.decompress()), _bits(mb))
        for q, p in zip(shadow.params, params):   # keep both on the same trajectory
            q.copy_(p.decompress())
    verify_buffer(buffer)


def test_adamw_compressed_moments_and_weights_follow_the_dense_trajectory():
    buffer = TensorBuffer(8 << 20)
    dense = _params(4)
    vector = torch.ones(257, dtype=torch.float32, device="cuda")
    a = [LCTTensor(dense[0].clone(), buffer, weight_dist), dense[1].clone(), vector.clone()]
    b = [dense[0].clone(), dense[1].clone(), vector.clone()]
    opt_a = SparseAdamW([dict(params=a[:2], lr=1e-2), dict(params=a[2:], lr=1e-3)], weight_decay=0.1,
                        compressed=True, buffer=buffer)
    opt_b = SparseAdamW([dict(params=b[:2], lr=1e-2), dict(params=b[2:], lr=1e-3)], weight_decay=0.1,
                        compressed=False)
    for step in range(3):
        grads = _grads(4, step)[:2] + [torch.full((257,), 1e-3 * (step + 1), device="cuda")]
        for pa, pb, g in zip(a, b, grads):
            pa.grad, pb.grad = g.clone(), g.clone()
        opt_a.step()
        opt_b.step()
        assert torch.equal(_bits(a[0].decompress()), _bits(b[0]))
        assert torch.equal(_bits(a[1]), _bits(b[1]))
        assert torch.equal(a[2], b[2])
        for pa, pb in zip(a, b):
            for key in ("exp_avg", "exp_avg_sq"):
                va, vb = opt_a.state[pa][key].value, opt_b.state[pb][key].value
                if pa.dtype == torch.bfloat16:
                    assert isinstance(va, LCTTensor)
                    assert torch.equal(_bits(va.decompress()), _bits(vb))
                else:
                    assert not isinstance(va, LCTTensor) and torch.equal(va, vb)
    verify_buffer(buffer)
