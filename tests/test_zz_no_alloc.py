"""lct_encode_noalloc: the encode entry point for callers that cannot allocate device memory.

A serving loop that forbids allocation after start-up, a process whose device memory all belongs
to another pool, or a plain C host has nowhere to get the two work buffers ``lct_encode`` wants
(one byte per stream, four ints per block).  ``lct_encode_noalloc`` keeps them in an array inside
the library instead and hands back only the overflow totals.  This test drives both entry points
through the C ABI on the same inputs and requires identical bytes - equal to each other and to
the CPU oracle's - twice in a row, the second time on a smaller tensor so that anything left in
the built-in array by the first call would show.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import tables_of
from losslessly_compressed_tensors_b200.codec.geometry import geometry
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType
from losslessly_compressed_tensors_b200.kernels import _lib
from synth import synth_bf16

MAX_BLOCKS = 1024  # stated limit of the built-in scratch


def _dev(array):
    return torch.from_numpy(np.ascontiguousarray(array).copy()).cuda()


def _encode_both(lib, bits, dist, center):
    """Run lct_encode + lct_scan_allocate and lct_encode_noalloc; return both result sets."""
    block_symbols, lanes, steps, fixed_words = geometry(dist)
    n = bits.size
    blocks = -(-n // block_symbols)
    size, streams = blocks * block_symbols, blocks * lanes
    encode_table, decode_table, _ = tables_of(dist)
    stream = torch.cuda.current_stream().cuda_stream
    src = _dev(bits)
    enc_t, dec_t = _dev(encode_table), _dev(decode_table)
    center_t = torch.tensor([center], dtype=torch.int32, device="cuda")
    shifted = torch.empty(256, dtype=torch.int32, device="cuda")
    assert lib.lct_shift_tables(enc_t.data_ptr(), dec_t.data_ptr(), center_t.data_ptr(),
                                shifted.data_ptr(), None, stream) == 0

    def outputs():
        return (torch.full((size,), 0xAB, dtype=torch.uint8, device="cuda"),
                torch.full((streams * fixed_words + 4,), -1, dtype=torch.int32, device="cuda"),
                torch.full((4,), -7, dtype=torch.int32, device="cuda"))

    side_a, payload_a, counts_a = outputs()
    extra = torch.empty(streams, dtype=torch.uint8, device="cuda")
    summaries = torch.empty(4 * blocks, dtype=torch.int32, device="cuda")
    assert lib.lct_encode(src.data_ptr(), side_a.data_ptr(), payload_a.data_ptr(), shifted.data_ptr(),
                          extra.data_ptr(), summaries.data_ptr(), size, n, block_symbols, steps,
                          fixed_words, 0, stream) == 0
    assert lib.lct_scan_allocate(summaries.data_ptr(), counts_a.data_ptr(), None, None, blocks, 256,
                                 stream) == 0

    side_b, payload_b, counts_b = outputs()
    assert lib.lct_encode_noalloc(src.data_ptr(), side_b.data_ptr(), payload_b.data_ptr(),
                                  shifted.data_ptr(), counts_b.data_ptr(), size, n, block_symbols,
                                  steps, fixed_words, 0, stream) == 0
    torch.cuda.synchronize()
    return (side_a, payload_a, counts_a), (side_b, payload_b, counts_b)


@pytest.mark.gpu
def test_noalloc_entry_point_matches_regular_encode_twice_in_a_row(oracle):
    lib = _lib.load()
    dist = Distribution(DistType.GAUSSIAN)
    # First call: several blocks, wide data (many overflow streams).  Second call: a smaller,
    # well-behaved tensor; stale scratch from the first call must not leak into its totals.
    calls = [(synth_bf16(5 * 32768 + 321, 901, "wide"), 0), (synth_bf16(32768 + 77, 902, "normal"), -1)]
    totals = []
    for bits, center in calls:
        regular, built_in = _encode_both(lib, bits, dist, center)
        for want, got, what in zip(regular, built_in, ("side bytes", "payload", "counts")):
            assert torch.equal(want, got), what          # bit-exact, as everywhere in this suite
        totals.append(built_in[2].tolist())
        # ... and both equal the CPU restatement of the reference's encoder and summary scan.
        encode_table, decode_table, rare = tables_of(dist)
        want = oracle.compress(bits, encode_table, decode_table, rare, geometry(dist), center=center)
        assert np.array_equal(built_in[0].cpu().numpy(), want["side"])
        assert np.array_equal(built_in[1].cpu().numpy(), want["encoded"])
        assert built_in[2].tolist()[:2] == [want["count"], want["tail_bytes"]]
    assert totals[0][0] > 0 and totals[0][1] > 0 and totals[0][2:] == [0, 0]
    assert totals[1][0] < totals[0][0]


@pytest.mark.gpu
def test_noalloc_entry_point_rejects_tensors_beyond_its_scratch():
    lib = _lib.load()
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: the size check comes first
    too_big = (MAX_BLOCKS + 1) * 32768
    code = lib.lct_encode_noalloc(fake, fake, fake, fake, fake, too_big, too_big, 32768, 128, 12, 0, None)
    assert code == -6
    assert b"1024" in lib.lct_error_string(code)
