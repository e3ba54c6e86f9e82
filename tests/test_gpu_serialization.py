"""Serialised compressed tensors (GPU): byte form -> tensor -> bit-exact values, in this process
and in another one that has nothing but the file."""
import hashlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from gpu_helpers import bits_of
from losslessly_compressed_tensors_b200 import config, sharded
from losslessly_compressed_tensors_b200.LCTensor import LCTTensor
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, NoiseLevel
from losslessly_compressed_tensors_b200.comp_tensor import CompressedTensor
from losslessly_compressed_tensors_b200.operations import compress, decompress
from losslessly_compressed_tensors_b200.serialization import (
    from_bytes, load_weight_set, save_weight_set, to_bytes)
from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer, _free_regions_snapshot

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _heavy(shape, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * torch.exp(torch.randn(shape, generator=g) * 4)
    return x.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("buffered", [True, False], ids=["arena", "private"])
@pytest.mark.parametrize("dist", [Distribution(DistType.LAPLACE, param=0.02),
                                  Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM),
                                  Distribution(DistType.LAPLACE, zero_prob=0.5, noise_level=NoiseLevel.SPARSE)],
                         ids=["laplace-clean", "gaussian-medium", "sparse"])
def test_byte_form_round_trip(buffered, dist):
    buffer = TensorBuffer(4 << 20) if buffered else None
    for shape, seed in (((300, 700), 1), ((70000,), 2), ((0, 4), 3), ((5,), 4)):
        x = _heavy(shape, seed)
        c = compress(x, dist, buffer)
        blob = c.to_bytes()
        assert blob[:8] == b"LCTENSOR" and len(blob) % 16 == 0
        back = CompressedTensor.from_bytes(blob)
        assert back.shape == tuple(shape) and back.distribution == dist
        assert back.buffer is None and back.stream_geometry == c.codec_geometry
        assert np.array_equal(bits_of(decompress(back)), bits_of(x))
        assert to_bytes(back) == blob                  # a fixed point: nothing is lost or reordered
        c.free()
    raw = compress(torch.ones(8, dtype=torch.bfloat16, device="cuda"), dist, buffer, allow_raw=True)
    assert torch.equal(decompress(from_bytes(raw.to_bytes())), decompress(raw))
    if buffered:
        assert _free_regions_snapshot(buffer) == [(0, 4 << 20)]


def test_records_are_checked():
    c = compress(_heavy((64, 1024), 5), Distribution(DistType.LAPLACE))
    blob = c.to_bytes()
    with pytest.raises(ValueError, match="not a LCTENSOR"):
        from_bytes(b"XXXXXXXX" + blob[8:])
    with pytest.raises(ValueError, match="version"):
        from_bytes(blob[:8] + (99).to_bytes(4, "little") + blob[12:])
    with pytest.raises(ValueError, match="truncated"):
        from_bytes(blob[:len(blob) // 2])
    config.lane_mapping = "linear"
    try:
        with pytest.raises(ValueError, match="lane mapping"):
            from_bytes(blob)
    finally:
        config.lane_mapping = "swizzle"
    lost = TensorBuffer(256)                          # far too small for this tensor's tails
    stranded = compress(_heavy((64, 1024), 6), Distribution(DistType.LAPLACE), lost)
    with pytest.raises(ValueError, match="never stored"):
        stranded.to_bytes()


def test_weight_set_file_decodes_in_another_process(tmp_path):
    """A file written here decodes bit-exactly in a fresh process that has only the file: no
    plan, no arena, no tensors of the writer."""
    shapes = sharded.gpt2_small_shapes(layers=1, d_model=256, vocab=1000)
    g = torch.Generator().manual_seed(9)
    buffer = TensorBuffer(8 << 20)
    dist = Distribution(DistType.EMPIRICAL)
    tensors, want = {}, {}
    for i, (name, shape) in enumerate(shapes):
        scale = 0.02 if i % 3 else 5.0
        x = (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()
        if i % 4 == 1:
            tensors[name] = LCTTensor(x, buffer, dist)                   # compressed, in an arena
        elif i % 4 == 2:
            tensors[name] = compress(x, Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.HIGH))
        else:
            tensors[name] = x                                           # dense: compressed on save
        want[name] = {"sha": hashlib.sha256(bits_of(x).tobytes()).hexdigest(), "shape": list(shape)}
    path = str(tmp_path / "weights.lct")
    written = save_weight_set(path, tensors, dist, buffer)
    assert written == os.path.getsize(path)
    here = load_weight_set(path, decode=True)
    assert list(here) == [name for name, _ in shapes]
    for name, x in here.items():
        assert hashlib.sha256(bits_of(x).tobytes()).hexdigest() == want[name]["sha"]
    result = subprocess.run([sys.executable, os.path.join(HERE, "serial_worker.py"), path, "swizzle"],
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    report = json.loads(result.stdout.strip().splitlines()[-1])
    assert list(report) == list(want)
    for name, entry in want.items():
        assert report[name]["sha"] == entry["sha"] and report[name]["shape"] == entry["shape"], name
    with pytest.raises(TypeError):
        save_weight_set(path, {"w": torch.zeros(4, device="cuda")})
