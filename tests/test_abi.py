"""The C-ABI library: it loads without a GPU, exports every symbol the header declares,
and rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from losslessly_compressed_tensors_b200.kernels import _lib


@pytest.fixture(scope="module")
def library():
    from losslessly_compressed_tensors_b200 import build

    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(library):
    header = open(os.path.join(ROOT, "include", "lct_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(lct_[a-z_]+)\s*\(", header))
    assert len(declared) >= 14
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert getattr(library, name) is not None, name


def test_identity_and_error_text(library):
    assert library.lct_version().decode().startswith("lct-b200 ")
    assert b"sm_100a" in library.lct_version()
    assert library.lct_error_string(0) == b"success"
    for code in (-1, -2, -3, -4, -5):
        assert library.lct_error_string(code) not in (b"", b"unknown lct error")


def test_argument_validation_needs_no_device(library):
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: validation fails first
    # geometry that is not a supported layout
    assert library.lct_encode(fake, fake, fake, fake, fake, fake, 65536, 65536, 65536, 100, 25, 0,
                              None) == -1
    # size not a whole number of blocks
    assert library.lct_encode(fake, fake, fake, fake, fake, fake, 1000, 1000, 65536, 256, 25, 0,
                              None) == -4
    # null pointers
    assert library.lct_encode(None, fake, fake, fake, fake, fake, 65536, 65536, 65536, 256, 25, 0,
                              None) == -2
    assert library.lct_scan_allocate(None, fake, None, None, 1, 256, None) == -2
    # misaligned payload
    odd = ctypes.c_void_p(0x1004)
    assert library.lct_encode(fake, fake, odd, fake, fake, fake, 65536, 65536, 65536, 256, 25, 0,
                              None) == -3
    operand = _lib.Operand()
    assert library.lct_decode(ctypes.byref(operand), fake, 65536, 65536, 65536, 256, 25, 8,
                              None) == -2
    assert library.lct_buffer_reset(fake, 3, 1024, None) == -4  # regions not a power of two
    assert library.lct_buffer_free(fake, None, fake, 256, None) == -2


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_library", None)
    monkeypatch.setattr(_lib, "LIBRARY_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()


def test_cpu_tensors_are_rejected():
    """No CPU path: the host API refuses anything that is not on a CUDA device."""
    import torch
    from losslessly_compressed_tensors_b200.kernels import dispatch

    with pytest.raises(ValueError, match="CUDA device"):
        dispatch.shift_decoding_table(torch.zeros(1024, dtype=torch.int32),
                                      torch.zeros(1, dtype=torch.int32))


def test_lane_mapping_switch_is_host_state_only():
    """lct_set_lane_mapping touches no device: it can be exercised without a GPU."""
    from losslessly_compressed_tensors_b200.kernels import _lib

    lib = _lib.load()
    assert lib.lct_get_lane_mapping() == 0            # "swizzle" is the default
    assert lib.lct_set_lane_mapping(1) == 0 and lib.lct_get_lane_mapping() == 1
    assert lib.lct_set_lane_mapping(2) != 0 and lib.lct_get_lane_mapping() == 1   # rejected, unchanged
    assert lib.lct_set_lane_mapping(0) == 0 and lib.lct_get_lane_mapping() == 0


def test_byte_form_framing_on_the_host():
    """to_bytes / from_bytes without a GPU: every field and component of a (fabricated) compressed
    tensor survives the round trip, arena-held overflow lists become private ones."""
    import numpy as np
    import torch

    from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType, StorageLayout
    from losslessly_compressed_tensors_b200.comp_tensor import CompressedTensor
    from losslessly_compressed_tensors_b200.serialization import from_bytes, to_bytes

    rng = np.random.default_rng(0)
    dist = Distribution(DistType.LAPLACE, param=0.02)
    blocks, count, tail = 2, 3, 40
    arena = torch.from_numpy(rng.integers(0, 255, 4096, dtype=np.uint8))
    c = CompressedTensor(
        torch.from_numpy(rng.integers(-2**31, 2**31 - 1, blocks * 256 * 25 + 4, dtype=np.int32)),
        blocks * 65536, torch.from_numpy(rng.integers(0, 255, blocks * 65536, dtype=np.uint8)),
        shape=(2, 60000), layout=StorageLayout.COMPRESSED, distribution=dist,
        stream_geometry=(65536, 256, 256, 25), center=torch.tensor([-7], dtype=torch.int32),
        decode_table=torch.arange(1024, dtype=torch.int32),
        fallback_count=torch.tensor([count], dtype=torch.int32),
        fallback_used=torch.tensor([tail], dtype=torch.int32),
        fallback_blocks=torch.arange(3 * blocks, dtype=torch.int32),
        fallback_descriptor=torch.tensor([1024, 48, 0, 1], dtype=torch.int32),
        fallback_buffer=arena)
    blob = to_bytes(c)
    back = from_bytes(blob, "cpu")
    assert back.shape == c.shape and back.size == c.size and back.distribution == dist
    assert back.stream_geometry == c.stream_geometry and int(back.center.item()) == -7
    for name in ("data", "sign_mantissa", "decode_table", "fallback_blocks", "fallback_count",
                 "fallback_used"):
        assert torch.equal(getattr(back, name), getattr(c, name)), name
    assert back.fallback_descriptor is None and back.buffer is None
    assert torch.equal(back.fallback_lanes, arena[1024:1027])
    assert torch.equal(back.fallback_starts, arena[1027:1030])
    assert torch.equal(back.fallback_buffer, arena[1030:1070])
    assert to_bytes(back) == blob
