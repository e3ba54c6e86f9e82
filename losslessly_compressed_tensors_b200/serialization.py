"""A self-describing byte form of compressed tensors, and weight-set files made of it.

The reference checkpoints dense tensors (``examples/nanogpt/train_gpt_lct.py:280-312`` decodes
every ``LCTTensor`` before ``torch.save``), so a checkpoint costs the dense bytes and a full
re-compression on load.  Here a ``CompressedTensor`` is written as it is:

    magic  b"LCTENSOR" | u32 version | u32 header bytes | header (JSON, UTF-8) | padding to 16
    | components, each starting on a 16-byte boundary

The header names everything a reader needs without the process, plan or arena that wrote the
bytes: lane mapping, stream geometry, the codebook (``Distribution`` fields), shape, layout,
exponent center, overflow counts and the offset, byte count and dtype of every component.
Overflow tails that lived in a shared arena are written as private lists (storage lane, first
overflow step, raw exponent tails), so a loaded tensor owns all its memory.  The codec bytes
(payload words, side bytes, per-block overflow metadata, shifted decode table) are exactly the
ones in device memory: a loaded tensor decodes through the same kernels, bit for bit.

A weight-set file is an index over such records:

    magic  b"LCTWSET\\0" | u32 version | u32 index bytes | index (JSON) | padding to 16 | records

Writing synchronises the host (the overflow counts are read); loading does not.
"""
from __future__ import annotations

import json
import struct
from typing import Mapping

import numpy as np
import torch

from . import config
from .comp_format import Distribution, DistType, NoiseLevel, StorageLayout
from .comp_tensor import CompressedTensor

TENSOR_MAGIC = b"LCTENSOR"
SET_MAGIC = b"LCTWSET\0"
VERSION = 1
_ALIGN = 16

_DTYPES = {"int32": (torch.int32, np.int32), "uint8": (torch.uint8, np.uint8),
           "bfloat16": (torch.bfloat16, np.uint16)}


def _pad(n: int) -> int:
    return -(-n // _ALIGN) * _ALIGN


def _host_bytes(tensor: torch.Tensor) -> bytes:
    flat = tensor.detach().contiguous().view(-1)
    if flat.dtype == torch.bfloat16:
        flat = flat.view(torch.int16)
    return flat.cpu().numpy().tobytes()


def _distribution_fields(d: Distribution) -> dict:
    return {"family": d.family.name, "param": d.param, "mean": d.mean,
            "zero_prob": d.zero_prob, "noise_level": d.noise_level.name}


def _distribution_of(fields: dict) -> Distribution:
    return Distribution(DistType[fields["family"]], param=fields["param"], mean=fields["mean"],
                        zero_prob=fields["zero_prob"], noise_level=NoiseLevel[fields["noise_level"]])


def _frame(magic: bytes, header: dict, parts: list[bytes]) -> bytes:
    """magic | version | header length | header | padding | parts (each padded to 16 bytes)."""
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    out = bytearray(magic + struct.pack("<II", VERSION, len(text)) + text)
    out.extend(b"\0" * (_pad(len(out)) - len(out)))
    for part in parts:
        out.extend(part)
        out.extend(b"\0" * (_pad(len(part)) - len(part)))
    return bytes(out)


def _unframe(magic: bytes, blob) -> tuple[dict, memoryview]:
    view = memoryview(blob)
    if len(view) < 16 or bytes(view[:8]) != magic:
        raise ValueError(f"not a {magic.decode('ascii', 'replace').strip(chr(0))} record")
    version, length = struct.unpack("<II", view[8:16])
    if version != VERSION:
        raise ValueError(f"unsupported format version {version} (this build reads {VERSION})")
    if 16 + length > len(view):
        raise ValueError("truncated header")
    header = json.loads(bytes(view[16:16 + length]).decode("utf-8"))
    return header, view[_pad(16 + length):]


def to_bytes(c: CompressedTensor) -> bytes:
    """The self-describing byte form of ``c`` (one host synchronisation)."""
    header = {
        "lane_mapping": config.lane_mapping, "layout": c.layout.name, "shape": list(c.shape),
        "size": int(c.size), "distribution": _distribution_fields(c.distribution),
    }
    parts: dict[str, tuple[bytes, str]] = {}
    if c.layout is StorageLayout.RAW:
        parts["dense"] = (_host_bytes(c.data), "bfloat16")
    else:
        count = int(c.fallback_count.item())
        tail_bytes = int(c.fallback_used.item())
        if c.fallback_descriptor is not None:
            offset, _, status, _ = (int(v) for v in c.fallback_descriptor.cpu().tolist())
            if count and status != 0:
                raise ValueError(f"the tensor's overflow tails were never stored (arena status "
                                 f"{status}): it cannot be decoded, so it is not written")
            region = (c.fallback_buffer[offset:offset + 2 * count + tail_bytes] if count
                      else c.fallback_buffer[:0])
            lanes, starts, tail = region[:count], region[count:2 * count], region[2 * count:]
        else:
            base = int(c.fallback_base)
            lanes, starts = c.fallback_lanes[:count], c.fallback_starts[:count]
            tail = c.fallback_buffer[base:base + tail_bytes]
        center = c.center
        header.update({
            "geometry": list(c.codec_geometry),
            "center": int(center.item()) if isinstance(center, torch.Tensor) else int(center),
            "overflow_count": count, "tail_bytes": tail_bytes,
        })
        parts["encoded"] = (_host_bytes(c.data), "int32")
        parts["side"] = (_host_bytes(c.sign_mantissa), "uint8")
        parts["decode_table"] = (_host_bytes(c.decode_table), "int32")
        parts["blocks"] = (_host_bytes(c.fallback_blocks), "int32")
        parts["lanes"] = (_host_bytes(lanes), "uint8")
        parts["starts"] = (_host_bytes(starts), "uint8")
        parts["tail"] = (_host_bytes(tail), "uint8")
    cursor, components = 0, {}
    for name, (data, dtype) in parts.items():
        components[name] = [cursor, len(data), dtype]       # offset from the first component
        cursor += _pad(len(data))
    header["components"] = components
    return _frame(TENSOR_MAGIC, header, [data for data, _ in parts.values()])


def from_bytes(blob, device: torch.device | str = "cuda") -> CompressedTensor:
    """Rebuild a ``CompressedTensor`` on ``device`` from ``to_bytes`` output (any bytes-like
    object; it is not modified).  The tensor owns private copies of everything, overflow lists
    included, and decodes with ``decompress`` like any other."""
    header, body = _unframe(TENSOR_MAGIC, blob)
    if header["lane_mapping"] != config.lane_mapping:
        raise ValueError(f"written with lane mapping {header['lane_mapping']!r}, but this process "
                         f"uses {config.lane_mapping!r} (set config.lane_mapping before loading)")
    device = torch.device(device)

    def component(name: str) -> torch.Tensor:
        offset, nbytes, dtype = header["components"][name]
        if offset + nbytes > len(body):
            raise ValueError(f"truncated record: component {name!r}")
        torch_dtype, numpy_dtype = _DTYPES[dtype]
        host = np.frombuffer(body[offset:offset + nbytes], dtype=numpy_dtype).copy()
        tensor = torch.from_numpy(host.view(np.int16) if dtype == "bfloat16" else host)
        if dtype == "bfloat16":
            tensor = tensor.view(torch.bfloat16)
        return tensor.to(device)

    distribution = _distribution_of(header["distribution"])
    shape = tuple(header["shape"])
    if header["layout"] == StorageLayout.RAW.name:
        return CompressedTensor(component("dense"), header["size"], distribution=distribution,
                                shape=shape, layout=StorageLayout.RAW)
    counts = torch.tensor([header["overflow_count"], header["tail_bytes"], 0, 0], dtype=torch.int32,
                          device=device)
    return CompressedTensor(
        component("encoded"), header["size"], component("side"),
        fallback_starts=component("starts"), fallback_lanes=component("lanes"),
        fallback_blocks=component("blocks"), fallback_buffer=component("tail"),
        fallback_descriptor=None, buffer=None, fallback_count=counts[:1],
        fallback_used=counts[1:2], distribution=distribution,
        center=torch.tensor([header["center"]], dtype=torch.int32, device=device),
        decode_table=component("decode_table"), shape=shape, layout=StorageLayout.COMPRESSED,
        stream_geometry=tuple(header["geometry"]),
    )


def _smaller_dense(tensor: torch.Tensor, distribution: Distribution) -> bool:
    """True when even an overflow-free encoding would take more bytes than the BF16 values
    (tensors much smaller than a codec block): such a tensor is written dense (RAW layout), the
    rule of ``compress(..., allow_raw=True)``."""
    from .codec.geometry import geometry

    block_symbols, lanes, _, fixed_words = geometry(distribution)
    blocks = -(-tensor.numel() // block_symbols)
    return blocks * block_symbols + (blocks * lanes * fixed_words + 4) * 4 > 2 * tensor.numel()


def save_weight_set(path, tensors: Mapping[str, object], distribution: Distribution | None = None,
                    buffer=None) -> int:
    """Write named tensors to ``path`` in compressed form; returns the bytes written.

    Values may be ``CompressedTensor``, ``LCTTensor`` (written as they are) or dense BF16 CUDA
    tensors (compressed with ``distribution`` first, all of them by one batched call when a
    ``buffer`` is given; tensors too small to gain anything are written dense).  Other dtypes are refused: this is the codec's file, not a pickle."""
    from .LCTensor import LCTTensor
    from .operations import compress_many, free_many

    names = list(tensors)
    values: list = [None] * len(names)
    dense_at, dense = [], []
    for i, name in enumerate(names):
        value = tensors[name]
        if isinstance(value, LCTTensor):
            values[i] = value.x
        elif isinstance(value, CompressedTensor):
            values[i] = value
        elif isinstance(value, torch.Tensor) and value.dtype == torch.bfloat16:
            if _smaller_dense(value, distribution or Distribution()):
                values[i] = CompressedTensor(value.detach().contiguous().view(-1), value.numel(),
                                             distribution=distribution or Distribution(),
                                             shape=tuple(value.shape), layout=StorageLayout.RAW)
            else:
                dense_at.append(i)
                dense.append(value)
        else:
            raise TypeError(f"{name}: expected a compressed tensor or a bfloat16 tensor")
    made = compress_many(dense, distribution or Distribution(), buffer) if dense else []
    for i, c in zip(dense_at, made):
        values[i] = c
    records = [to_bytes(c) for c in values]
    free_many(made)
    index, cursor = [], 0
    for name, record in zip(names, records):
        index.append({"name": name, "offset": cursor, "nbytes": len(record)})
        cursor += _pad(len(record))
    blob = _frame(SET_MAGIC, {"tensors": index}, records)
    with open(path, "wb") as handle:
        handle.write(blob)
    return len(blob)


def load_weight_set(path, device: torch.device | str = "cuda", *,
                    decode: bool = False) -> dict:
    """Read a file written by ``save_weight_set``: name -> ``CompressedTensor`` on ``device``
    (or, with ``decode``, name -> dense BF16 tensor, decoded by one launch per codebook)."""
    from .operations import decompress_many

    with open(path, "rb") as handle:
        blob = handle.read()
    header, body = _unframe(SET_MAGIC, blob)
    loaded = {}
    for entry in header["tensors"]:
        start, stop = entry["offset"], entry["offset"] + entry["nbytes"]
        if stop > len(body):
            raise ValueError(f"truncated file: tensor {entry['name']!r}")
        loaded[entry["name"]] = from_bytes(body[start:stop], device)
    if not decode:
        return loaded
    return dict(zip(loaded, decompress_many(list(loaded.values()))))
