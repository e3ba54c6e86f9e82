"""The compiled reference on the same GPU, as the bit oracle of the fused float path, and the
reference's own callers running unmodified on this library.

Both need a copy of the reference checkout under ``baseline/_ref`` (``__graft_entry__.build()``
makes it where the checkout exists; it is not part of this repository) and are skipped without
it.  Everything that imports the reference runs in a process of its own
(``tests/reference_runner.py``): the reference and this library cannot both be ``LCT``.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import reference_runner
from helpers import oracle_compress
from gpu_helpers import bits_of, host
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not reference_runner.available(),
                                 reason="no copy of the reference checkout under baseline/_ref")]

RUNNER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_runner.py")


def _run(mode, out, *extra, timeout=900):
    done = subprocess.run([sys.executable, RUNNER, mode, "--out", str(out), *extra],
                          capture_output=True, text=True, timeout=timeout)
    assert done.returncode == 0, f"reference_runner {mode} failed:\n{done.stdout[-2000:]}\n{done.stderr[-4000:]}"


def test_config4_recurrence_matches_the_compiled_reference(oracle, tmp_path):
    """BASELINE configuration 4 (m = 0.95 m + g on compressed momentum, 20 steps): decoded bits
    and every compressed component, step by step, against the reference's own fused path
    (``LCTTensor.mul_add_`` -> ``pointwise_compressed_dense``, compiled by Triton on this GPU).
    The reference leaves payload words past a lane's last written word unset, so the payload is
    compared on the words the format defines (the oracle marks them)."""
    out = tmp_path / "reference_bits.npz"
    sizes = ("1024x1024", "4096x4096")
    steps = 20
    _run("bits", out, "--sizes", ",".join(sizes), "--steps", str(steps))
    want = np.load(out)
    dist = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    buffer = TensorBuffer(64 << 20)
    for index, size in enumerate(sizes):
        rows, cols = (int(v) for v in size.split("x"))
        momentum, grads = reference_runner.config4_inputs(rows, cols, steps)
        state = LCTTensor(momentum.cuda(), buffer, dist)
        for step, grad in enumerate(grads):
            state.mul_add_(alpha, grad.cuda())
            c = state.x
            dense = state.decompress()
            key = f"{size}_{step}"
            what = f"{size} step {step}"
            assert reference_runner._sha(dense.view(torch.int16)) == str(want["dense_sha_" + key]), what
            assert reference_runner._sha(c.sign_mantissa) == str(want["side_sha_" + key]), what
            assert int(c.center.item()) == int(want["center_" + key]), what
            assert int(c.fallback_count.item()) == int(want["count_" + key]), what
            assert int(c.fallback_used.item()) == int(want["used_" + key]), what
            assert int(c.memory_size()) == int(want["memory_size_" + key]), what
            assert reference_runner._sha(c.decode_table) == str(want["decode_table_sha_" + key]), what
            if index == 0:
                defined = oracle_compress(oracle, bits_of(dense), dist, None)["defined"].astype(bool)
                ours, theirs = host(c.data), want["payload_" + key]
                assert ours.shape == theirs.shape, what
                assert np.array_equal(ours[defined], theirs[defined]), what
        state.free()


def test_reference_callers_run_unmodified_on_this_library(tmp_path):
    """``examples/benchmarks/benchmark_lct.py`` (its ``run_case``: round trip and ratio ceiling
    for all five cases), ``benchmark_pointwise.py`` (its ``check_result`` on every fused operation
    with dense and compressed output), ``LCT/components/layers.py`` and ``mlps.py`` (``Relu2Linear``,
    the shared-input Q/K/V projection, ``RMSNormFunction``, ``FlashAttention``, ``FFN``, ``RMSFFN``, and the
    reference's own optimizers ``SparseMuon`` / ``SparseAdamW`` / ``SparseSGDM`` with their state compressed
    by this library; ``RMSLinear`` forward and
    backward with the saved activation compressed) on ``compat.install_as_lct()``."""
    out = tmp_path / "dropin.json"
    _run("dropin", out)
    report = json.loads(out.read_text())
    assert report["benchmark_lct_cases"] == 5
    assert report["benchmark_pointwise_checks"] == 10
    assert "identical" in report["rms_linear"]
    for layer in ("relu2_linear", "rms_norm_qkv", "rms_norm_function", "ffn"):
        assert "identical" in report[layer], layer
    for optional in ("rms_ffn", "flash_attention"):     # need operators of the installed PyTorch
        assert "identical" in report[optional] or report[optional].startswith("not run"), report[optional]
    assert "identical" in report["reference_muon"] and "identical" in report["reference_adamw"]
    assert report["reference_sgdm"] == "three fused steps"
    print({k: v[:40] for k, v in report.items() if isinstance(v, str)})


def test_each_codec_decodes_what_the_other_compressed(tmp_path):
    """Payload interchange on the GPU: this library's compressed tensors decode bit-exactly
    through the reference's kernels (its generic decoder and, where it builds, its A100 decoder,
    ``LCT/kernels/a100/decode.py:13-15``: "payloads are interchangeable") and the reference's
    through this library's, private and arena-held overflow, every layout, ragged sizes; and
    both report the same ``memory_size()``."""
    out = tmp_path / "interchange.json"
    _run("interchange", out)
    with open(out) as handle:
        report = json.load(handle)
    generic = {k: v for k, v in report["cases"].items() if k.startswith("generic/")}
    assert len(generic) == 12
    assert any(v["overflow_streams"] > 0 for v in generic.values())
    for key, result in report["cases"].items():
        assert result["reference_decodes_ours"], key
        assert result["this_decodes_reference"], key
        assert result["same_memory_size"], key
    print("A100 decoder of the reference:", report["a100"],
          sum(k.startswith("a100/") for k in report["cases"]), "cases")
