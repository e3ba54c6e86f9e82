"""Regenerate the golden fixtures by running the UNMODIFIED reference on the CPU.

    python tests/golden/make_golden.py            # writes tables.npz, codec.json
    LCT_GOLDEN_LANE_MAPPING=linear python tests/golden/make_golden.py linear   # adds the linear-mapping cases

Needs the reference checkout (its location: ``LCT_REFERENCE_ROOT``, see ``reference_shim``)
and runs its Triton kernels under ``TRITON_INTERPRET=1`` through
``reference_shim``; that takes a few minutes.  The test-suite only reads the
files written here and never imports the reference.

What is recorded, per case: a digest of the synthetic input, the sampled
center, ``memory_size()``, every small component in full (overflow lanes,
starts, tails, block metadata, allocator descriptor) and SHA-256 digests of the
large ones (payload words, side bytes, shifted decode table, decoded output).

The reference allocates its outputs with ``torch.empty`` and leaves payload
words past a lane's end (and side bytes of padding) unwritten.  To get
reproducible bytes each encode is run twice with those allocations pre-filled
with 0x00 and with 0xFF: words equal in both runs are the ones the reference
defines (recorded as a bit mask digest), and the 0x00 run is the byte-exact
target for an encoder that zero-fills.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import reference_shim  # noqa: E402,F401  (must precede any LCT import)
import numpy as np  # noqa: E402
import torch  # noqa: E402

from synth import synth_bf16, synth_exact_scale  # noqa: E402

import LCT.codec.encode as ref_encode  # noqa: E402
import LCT.codec.pointwise as ref_pointwise  # noqa: E402
import LCT.codec.decode as ref_decode  # noqa: E402
from LCT.comp_format import Distribution, DistType, NoiseLevel  # noqa: E402
from LCT.compression.huffman_tables import _get_distribution_tables  # noqa: E402
from LCT.operations import (  # noqa: E402
    a_compA_add_B, a_compA_add_b_B, a_compA_add_compB, compress, decompress,
)
from LCT.tensor_buffer import TensorBuffer, _free_regions_snapshot  # noqa: E402


class _FilledTorch:
    """Stands in for the ``torch`` global of a reference module: ``empty`` returns
    memory pre-filled with a chosen byte instead of whatever the heap held."""

    fill = 0

    def __getattr__(self, name):
        return getattr(torch, name)

    def empty(self, *args, **kwargs):
        out = torch.zeros(*args, **kwargs)
        if _FilledTorch.fill and out.numel():
            out.view(torch.uint8).fill_(_FilledTorch.fill)
        return out

    def empty_like(self, other, **kwargs):
        out = torch.zeros_like(other, **kwargs)
        if _FilledTorch.fill and out.numel():
            out.view(torch.uint8).fill_(_FilledTorch.fill)
        return out


for _module in (ref_encode, ref_pointwise, ref_decode):
    _module.torch = _FilledTorch()


def sha(array) -> str:
    if isinstance(array, torch.Tensor):
        array = array.contiguous().view(torch.uint8).numpy()
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()[:32]


def full_or_digest(tensor, limit=2048):
    values = tensor.reshape(-1).tolist()
    return values if len(values) <= limit else {"sha": sha(tensor), "len": len(values)}


TABLE_CASES = [
    ("GAUSSIAN", 1.0, 0.0, 0.0), ("LAPLACE", 0.25, 0.0, 0.0), ("LAPLACE", 1.0, 0.0, 0.5),
    ("EMPIRICAL", 1.0, 0.0, 0.0), ("EMPIRICAL", 1.0, 0.0, 0.02), ("GAMMA", 1.0, 0.0, 0.0),
    ("GAUSSIAN", 2.0, 50.0, 0.0), ("LAPLACE", 1.5, 0.0, 0.0), ("GAUSSIAN", 1.0, 0.0, 0.3),
    ("EMPIRICAL", 2.0, 1.0, 0.1),
]


def make_tables():
    out = {}
    for family, param, mean, zero_prob in TABLE_CASES:
        encode, decode, rare = _get_distribution_tables(DistType[family], param, mean, zero_prob)
        key = f"{family}|{param}|{mean}|{zero_prob}"
        out[key + "|encode"] = encode.numpy().astype(np.int32)
        out[key + "|decode"] = decode.numpy().astype(np.int32)
        out[key + "|rare"] = np.array([rare], np.int32)
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **out)
    print("tables:", len(TABLE_CASES))


def dist_of(spec) -> Distribution:
    return Distribution(DistType[spec["family"]], param=spec.get("param", 1.0),
                        mean=spec.get("mean", 0.0), zero_prob=spec.get("zero_prob", 0.0),
                        noise_level=NoiseLevel[spec.get("noise", "CLEAN")])


def describe(c, buffer) -> dict:
    """Everything observable on a reference CompressedTensor."""
    blocks = c.fallback_blocks.numel() // 3
    record = {
        "geometry": list(c.stream_geometry), "size": c.size, "center": int(c.center.item()),
        "memory_size": c.memory_size(), "count": int(c.fallback_count.item()),
        "tail_bytes": int(c.fallback_used.item()),
        "encoded_sha": sha(c.data), "encoded_len": c.data.numel(),
        "side_sha": sha(c.sign_mantissa), "decode_table_sha": sha(c.decode_table),
        "blocks": full_or_digest(c.fallback_blocks), "n_blocks": blocks,
    }
    count, tail_bytes = record["count"], record["tail_bytes"]
    if c.fallback_descriptor is None:
        record["lanes"] = full_or_digest(c.fallback_lanes)
        record["starts"] = full_or_digest(c.fallback_starts)
        record["tail"] = full_or_digest(c.fallback_buffer)
    else:
        descriptor = c.fallback_descriptor.tolist()
        record["descriptor"] = descriptor
        base = descriptor[0]
        if descriptor[2] == 0:
            arena = buffer.data
            record["lanes"] = full_or_digest(arena[base:base + count])
            record["starts"] = full_or_digest(arena[base + count:base + 2 * count])
            record["tail"] = full_or_digest(arena[base + 2 * count:base + 2 * count + tail_bytes])
        record["free_regions"] = _free_regions_snapshot(buffer)
    return record


def encode_twice(make):
    """Run ``make()`` with 0x00- and 0xFF-filled scratch; return the 0x00 result and
    the masks of payload words / side bytes that the reference actually writes."""
    _FilledTorch.fill = 0xFF
    ones = make()
    _FilledTorch.fill = 0
    zeros = make()
    word_mask = (zeros.data == ones.data).numpy()
    side_mask = (zeros.sign_mantissa == ones.sign_mantissa).numpy()
    return zeros, ones, word_mask, side_mask


CODEC_CASES = [
    dict(name="gauss_clean_ragged", n=40000, kind="normal", seed=1, family="GAUSSIAN"),
    dict(name="gauss_clean_wide", n=32768 + 5000, kind="wide", seed=2, family="GAUSSIAN"),
    dict(name="laplace_clean_outliers", n=65536 + 1000, kind="outliers", seed=3, base=-6,
         family="LAPLACE", param=0.02),
    dict(name="sparse_buffered", n=70000, kind="sparse", seed=4, family="LAPLACE", zero_prob=0.5,
         noise="SPARSE", buffer=1 << 20),
    dict(name="medium_small_values", n=33000, kind="normal", seed=5, base=-10, family="GAUSSIAN",
         noise="MEDIUM"),
    dict(name="high_wide_buffered", n=32768 * 2, kind="wide", seed=6, family="EMPIRICAL",
         noise="HIGH", buffer=1 << 20),
    dict(name="empirical_tiny_3072", n=3072, kind="normal", seed=7, base=-6, family="EMPIRICAL"),
    dict(name="one_element", n=1, kind="normal", seed=8, family="GAUSSIAN"),
    dict(name="n255", n=255, kind="laplace", seed=9, family="LAPLACE"),
    dict(name="n256", n=256, kind="wide", seed=10, family="GAUSSIAN"),
    dict(name="n257", n=257, kind="wide", seed=11, family="GAUSSIAN"),
    dict(name="all_ones", n=768, kind="ones", seed=12, family="EMPIRICAL"),
    dict(name="all_zeros", n=768, kind="zeros", seed=13, family="EMPIRICAL"),
    dict(name="gamma_clean", n=20000, kind="sparse", seed=14, family="GAMMA"),
    dict(name="gauss_mean_shift", n=9000, kind="normal", seed=15, base=5, family="GAUSSIAN",
         param=2.0, mean=50.0),
    dict(name="block_minus_one", n=32767, kind="wide", seed=16, family="GAUSSIAN"),
    dict(name="block_plus_one", n=32769, kind="laplace", seed=17, family="GAUSSIAN"),
]


# Subsets recorded a second time with ``config.lane_mapping = "linear"`` (a run of its own:
# ``LCT_GOLDEN_LANE_MAPPING=linear python tests/golden/make_golden.py linear``).
LINEAR_CODEC = ("gauss_clean_wide", "laplace_clean_outliers", "sparse_buffered",
                "medium_small_values", "high_wide_buffered", "n257", "block_plus_one")
LINEAR_POINTWISE = ("scale_exact_wide_buffered", "two_scale_exact_medium", "dual_exact_buffered")


def make_codec(only=None):
    cases = []
    for spec in CODEC_CASES:
        if only is not None and spec["name"] not in only:
            continue
        t0 = time.time()
        bits = synth_bf16(spec["n"], spec["seed"], spec["kind"], spec.get("base", 0))
        x = torch.from_numpy(bits.copy()).view(torch.bfloat16)
        dist = dist_of(spec)
        buffer = TensorBuffer(spec["buffer"], device="cpu") if "buffer" in spec else None

        def make():
            if buffer is not None:
                buffer.reset()
                buffer.data.zero_()
            return compress(x, dist, buffer)

        c, c_ones, word_mask, side_mask = encode_twice(make)
        restored = decompress(c)
        assert torch.equal(restored.view(torch.int16), x.view(torch.int16)), spec["name"]
        record = dict(spec)
        record["input_sha"] = sha(bits)
        record.update(describe(c, buffer))
        record["word_mask_sha"] = sha(np.packbits(word_mask))
        record["word_mask_count"] = int(word_mask.sum())
        record["side_mask_sha"] = sha(np.packbits(side_mask))
        record["side_mask_count"] = int(side_mask.sum())
        record["decoded_sha"] = sha(restored)
        if buffer is not None:
            c.free()
            record["free_regions_after_free"] = _free_regions_snapshot(buffer)
        cases.append(record)
        print(f"{spec['name']:28s} center={record['center']:4d} count={record['count']:4d} "
              f"tail={record['tail_bytes']:6d} mem={record['memory_size']:8d} {time.time() - t0:5.1f}s")
    return cases


# Fused operations whose results are exact (no rounding happens), so the Triton
# interpreter's truncating float->bf16 cast cannot change them.  Only the
# float32 "scaled" operations are used: the interpreter's native bf16 add and
# multiply do not produce usable values at all.
POINTWISE_CASES = [
    dict(name="scale_exact_private", n=40000, kind="normal", seed=21, family="GAUSSIAN",
         op="scale", alpha=2.0),
    dict(name="scale_exact_wide_buffered", n=32768 + 777, kind="wide", seed=22, family="GAUSSIAN",
         op="scale", alpha=0.5, buffer=1 << 20),
    dict(name="two_scale_exact_medium", n=33000, kind="normal", seed=23, base=-10,
         family="GAUSSIAN", noise="MEDIUM", op="two_scale", alpha=0.0, beta=0.5),
    dict(name="dual_exact_private", n=32768 + 123, kind="wide", seed=24, family="GAUSSIAN",
         op="dual", alpha=4.0),
    dict(name="dual_exact_buffered", n=65536 + 5, kind="outliers", seed=25, base=-3,
         family="LAPLACE", op="dual", alpha=-0.5, buffer=1 << 20),
]


def make_pointwise(only=None):
    cases = []
    for spec in POINTWISE_CASES:
        if only is not None and spec["name"] not in only:
            continue
        t0 = time.time()
        bits = synth_bf16(spec["n"], spec["seed"], spec["kind"], spec.get("base", 0))
        x = torch.from_numpy(bits.copy()).view(torch.bfloat16)
        dist = dist_of(spec)
        buffer = TensorBuffer(spec["buffer"], device="cpu") if "buffer" in spec else None
        _FilledTorch.fill = 0
        a = compress(x, dist, buffer)
        record = dict(spec)
        record["input_sha"] = sha(bits)
        if spec["op"] == "two_scale":
            other_bits = synth_exact_scale(spec["n"], spec["seed"] + 100)
            other = torch.from_numpy(other_bits.copy()).view(torch.bfloat16)
            alpha = torch.tensor([spec["alpha"]], dtype=torch.float32)
            beta = torch.tensor([spec["beta"]], dtype=torch.float32)
            dense = a_compA_add_b_B(a, alpha, other, beta)
            expect = (other.float() * spec["beta"]).to(torch.bfloat16)
            comp = a_compA_add_b_B(a, alpha, other, beta, dense_output=False, buffer=buffer)
            record["other_sha"] = sha(other_bits)
        elif spec["op"] == "scale":
            other = torch.zeros(spec["n"], dtype=torch.bfloat16)
            alpha = torch.tensor([spec["alpha"]], dtype=torch.float32)
            dense = a_compA_add_B(a, alpha, other)
            expect = (x.float() * spec["alpha"]).to(torch.bfloat16)
            comp = a_compA_add_B(a, alpha, other, dense_output=False, buffer=buffer)
        else:
            zero = compress(torch.zeros(spec["n"], dtype=torch.bfloat16), dist, buffer)
            alpha = torch.tensor([spec["alpha"]], dtype=torch.float32)
            dense = a_compA_add_compB(a, alpha, zero)
            expect = (x.float() * spec["alpha"]).to(torch.bfloat16)
            comp = a_compA_add_compB(a, alpha, zero, dense_output=False, buffer=buffer)
        assert torch.equal(dense.view(torch.int16), expect.view(torch.int16)), spec["name"]
        assert torch.equal(decompress(comp).view(torch.int16), expect.view(torch.int16)), spec["name"]
        record["dense_sha"] = sha(dense)
        record["result"] = describe(comp, buffer)
        cases.append(record)
        print(f"{spec['name']:28s} center={record['result']['center']:4d} "
              f"count={record['result']['count']:4d} {time.time() - t0:5.1f}s")
    return cases


def make_allocator():
    """Drive the reference allocator kernels through a fixed request script."""
    buffer = TensorBuffer(4096, max_free_regions=8, device="cpu")
    live, trace = {}, []
    script = [("alloc", 100), ("alloc", 16), ("alloc", 1000), ("alloc", 0), ("free", 1), ("alloc", 8),
              ("alloc", 5000), ("free", 0), ("free", 2), ("alloc", 2000), ("free", 0)]
    script += [("alloc", 48)] * 16                          # steps 11..26
    script += [("free", k) for k in range(11, 27, 2)]       # fragment until the list is full
    script += [("free", 12), ("free", 14), ("alloc", 96), ("alloc", 4096), ("reset", 0),
               ("free", 16), ("alloc", 4096), ("alloc", 1), ("free", 41)]
    for step, (what, arg) in enumerate(script):
        entry = {"op": what, "arg": arg}
        if what == "alloc":
            allocation = buffer.allocate(torch.tensor([arg], dtype=torch.int32))
            live[step] = allocation
            entry["descriptor"] = allocation.descriptor.tolist()
        elif what == "free":
            status = buffer.free(live[arg])
            entry["status"] = int(status.item())
            entry["descriptor"] = live[arg].descriptor.tolist()
        else:
            buffer.reset()
        entry["free_regions"] = _free_regions_snapshot(buffer)
        trace.append(entry)
    return {"capacity": 4096, "max_free_regions": 8, "trace": trace}


def make_config1():
    """BASELINE configuration 1: 1024x1024 N(0,1) from torch's CPU generator, seed 0."""
    t0 = time.time()
    torch.manual_seed(0)
    x = torch.randn(1024, 1024).to(torch.bfloat16)
    dist = Distribution(DistType.GAUSSIAN)
    c, _, word_mask, side_mask = encode_twice(lambda: compress(x, dist))
    restored = decompress(c)
    assert torch.equal(restored.view(torch.int16), x.view(torch.int16))
    record = {"name": "config1_randn_seed0", "shape": [1024, 1024], "family": "GAUSSIAN",
              "input_sha": sha(x), "word_mask_count": int(word_mask.sum()),
              "word_mask_sha": sha(np.packbits(word_mask))}
    record.update(describe(c, None))
    print(f"config1 center={record['center']} count={record['count']} mem={record['memory_size']} "
          f"{time.time() - t0:5.1f}s")
    return record


def main():
    which = set(sys.argv[1:]) or {"tables", "codec", "pointwise", "allocator", "config1"}
    mapping = os.environ.get("LCT_GOLDEN_LANE_MAPPING", "swizzle")
    if ("linear" in which) != (mapping == "linear") or ("linear" in which and len(which) > 1):
        raise SystemExit("the linear fixtures are a run of their own: "
                         "LCT_GOLDEN_LANE_MAPPING=linear python make_golden.py linear")
    if "tables" in which:
        make_tables()
    path = os.path.join(HERE, "codec.json")
    data = json.load(open(path)) if os.path.exists(path) else {}
    if "codec" in which:
        data["codec"] = make_codec()
    if "pointwise" in which:
        data["pointwise"] = make_pointwise()
    if "allocator" in which:
        data["allocator"] = make_allocator()
    if "config1" in which:
        data["config1"] = make_config1()
    if "linear" in which:
        data["codec_linear"] = make_codec(LINEAR_CODEC)
        data["pointwise_linear"] = make_pointwise(LINEAR_POINTWISE)
    data["generator"] = {"torch": torch.__version__, "numpy": np.__version__,
                         "note": "reference run under TRITON_INTERPRET=1 on CPU"}
    with open(path, "w") as handle:
        json.dump(data, handle, indent=1, sort_keys=True)
    print("wrote", path)


if __name__ == "__main__":
    main()
