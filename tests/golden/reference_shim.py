"""Load the unmodified reference (a Python/Triton project) on a GPU-less host.

Only the fixture generator in this directory imports this module; nothing in
the test-suite or the product does.  It makes four adjustments at import time
and never edits the reference's files:

1. the reference targets Python 3.14's deferred annotations, so a source
   loader prepends ``from __future__ import annotations`` to its modules;
2. its autotune module asks for a CUDA device at import, so the device probe
   is replaced and a single-config tuning profile is selected;
3. its layout helpers are jitted functions that need ``tl`` in their globals
   when run under the Triton interpreter;
4. table tensors and backend selection are pointed at the CPU.

Run with ``TRITON_INTERPRET=1`` (set here if unset): integer codec paths are
exact under the interpreter; its float->bf16 casts truncate, so float results
of the fused operations are NOT taken from it.
"""
import importlib.machinery
import os
import sys

REFERENCE_ROOT = os.environ.get("LCT_REFERENCE_ROOT", "/root/reference")
os.environ.setdefault("TRITON_INTERPRET", "1")
sys.path.insert(0, REFERENCE_ROOT)

_FUTURE = "from __future__ import annotations"


class _DeferredAnnotationsLoader(importlib.machinery.SourceFileLoader):
    def source_to_code(self, data, path, *, _optimize=-1):
        text = data.decode() if isinstance(data, bytes) else data
        if path.startswith(REFERENCE_ROOT) and _FUTURE not in text:
            stripped = text.lstrip()
            if stripped.startswith(('"""', "'''")):
                quote = stripped[:3]
                end = text.index(quote, text.index(quote) + 3) + 3
                text = text[:end] + ";" + _FUTURE + text[end:]
            else:
                text = _FUTURE + ";" + text
        return super().source_to_code(text, path, _optimize=_optimize)


class _ReferenceFinder(importlib.machinery.PathFinder):
    @classmethod
    def find_spec(cls, name, path=None, target=None):
        if name != "LCT" and not name.startswith("LCT."):
            return None
        spec = importlib.machinery.PathFinder.find_spec(name, path, target)
        if spec is not None and spec.origin and spec.origin.endswith(".py"):
            spec.loader = _DeferredAnnotationsLoader(name, spec.origin)
        return spec


sys.meta_path.insert(0, _ReferenceFinder)

import torch  # noqa: E402
import triton.language as tl  # noqa: E402
from LCT import config  # noqa: E402

config.kernel_backend = "5090"  # one launch config per kernel: no autotune timing runs

if not torch.cuda.is_available():
    import LCT.kernels.device as _device

    _device.device_profile = lambda device=None: _device.DeviceProfile(
        model="generic", family="generic")

    import LCT.compression.huffman_tables as _tables

    class _CpuTorch:
        def __getattr__(self, name):
            return getattr(torch, name)

        def tensor(self, *args, **kwargs):
            kwargs.pop("device", None)
            return torch.tensor(*args, **kwargs)

    _tables.torch = _CpuTorch()

    import LCT.kernels.backends as _backends
    import LCT.kernels.dispatch as _dispatch

    _backends.backend_for = _dispatch.backend_for = lambda device: _backends.TRITON

import LCT.kernels.generic.layout as _layout  # noqa: E402

_layout.tl = tl
