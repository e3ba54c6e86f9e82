"""Host-side codebook construction against tables produced by the reference itself."""
import numpy as np
import pytest

from losslessly_compressed_tensors_b200.codec.geometry import geometry
from losslessly_compressed_tensors_b200.comp_format import (
    Distribution, DistType, NoiseLevel, StorageLayout,
)
from losslessly_compressed_tensors_b200.compression.huffman_tables import (
    FIRST_BITS, FIRST_MASK, _canonical_codes, _length_limited_huffman_lengths, host_tables,
)


def test_tables_match_reference(golden_tables):
    keys = sorted({k.rsplit("|", 1)[0] for k in golden_tables.files})
    assert len(keys) >= 10
    for key in keys:
        family, param, mean, zero_prob = key.split("|")
        encode, decode, rare = host_tables(DistType[family], float(param), float(mean),
                                           float(zero_prob))
        assert np.array_equal(encode, golden_tables[key + "|encode"]), key
        assert np.array_equal(decode, golden_tables[key + "|decode"]), key
        assert rare == int(golden_tables[key + "|rare"][0]), key


def test_table_structure():
    encode, decode, rare = host_tables(DistType.GAUSSIAN, 1.0, 0.0, 0.0)
    assert encode.shape == (256,) and decode.shape == (1 << FIRST_BITS,)
    lengths = encode >> 20
    direct = lengths <= 8
    assert rare == 8 and lengths[~direct].tolist() == [16] * int((~direct).sum())
    # Every direct code decodes to its own index through the first-level table.
    for index in np.nonzero(direct)[0]:
        code = int(encode[index]) & 0xFFFFF
        entry = int(decode[code & FIRST_MASK])
        assert entry & 255 == lengths[index] and (entry >> 8) & 255 == index
    # Kraft equality: the code is complete.
    esc = {int(encode[i]) & ((1 << rare) - 1) for i in np.nonzero(~direct)[0]}
    assert len(esc) == 1
    kraft = sum(2.0 ** -int(l) for l in lengths[direct]) + 2.0 ** -rare
    assert abs(kraft - 1.0) < 1e-12


def test_package_merge_small_cases():
    assert _length_limited_huffman_lengths([1, 1], 8).tolist() == [1, 1]
    assert _length_limited_huffman_lengths([1, 1, 2], 8).tolist() == [2, 2, 1]
    limited = _length_limited_huffman_lengths([1, 2, 4, 8, 16, 32], 3)
    assert limited.max() <= 3 and abs(sum(2.0 ** -int(l) for l in limited) - 1.0) < 1e-12
    with pytest.raises(ValueError):
        _length_limited_huffman_lengths([0, 0, 0], 8)
    codes = _canonical_codes([2, 1, 2])
    assert codes == {1: (0, 1), 0: (2, 2), 2: (3, 2)}


def test_distribution_validation_and_rounding():
    d = Distribution(DistType.LAPLACE, param=0.02)
    assert d.param == 0.25 and d.mean == 0.0 and d.zero_prob == 0.0
    assert Distribution(DistType.GAUSSIAN, param=1.13, mean=0.4, zero_prob=None).param == 1.25
    assert Distribution(mean=0.4).mean == 0.5
    assert Distribution(zero_prob=0.123).zero_prob == 0.12
    assert str(Distribution(DistType.GAUSSIAN)) == "gaussian/std=1.0/mean=0.0/clean"
    with pytest.raises(TypeError):
        Distribution("gaussian")
    with pytest.raises(TypeError):
        Distribution(noise_level="clean")
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(ValueError):
            Distribution(param=bad)
    with pytest.raises(ValueError):
        Distribution(mean=float("inf"))
    for bad in (-0.1, 1.5, float("nan")):
        with pytest.raises(ValueError):
            Distribution(zero_prob=bad)
    assert [m.name for m in NoiseLevel] == ["CLEAN", "MEDIUM", "HIGH", "SPARSE"]
    assert StorageLayout.RAW.value == 1 and StorageLayout.COMPRESSED.value == 2


def test_geometry_matches_reference_layouts():
    expect = {
        (DistType.EMPIRICAL, NoiseLevel.CLEAN): (65536, 256, 256, 25),
        (DistType.LAPLACE, NoiseLevel.CLEAN): (65536, 256, 256, 25),
        (DistType.GAUSSIAN, NoiseLevel.CLEAN): (32768, 256, 128, 12),
        (DistType.LAPLACE, NoiseLevel.SPARSE): (65536, 256, 256, 20),
        (DistType.GAUSSIAN, NoiseLevel.SPARSE): (65536, 256, 256, 20),
        (DistType.GAUSSIAN, NoiseLevel.MEDIUM): (32768, 256, 128, 19),
        (DistType.EMPIRICAL, NoiseLevel.HIGH): (32768, 256, 128, 22),
    }
    for (family, level), want in expect.items():
        assert geometry(Distribution(family, noise_level=level)) == want
