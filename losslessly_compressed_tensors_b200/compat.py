"""Make this package importable under the reference's name.

    import losslessly_compressed_tensors_b200.compat as compat
    compat.install_as_lct()
    from LCT.operations import compress, decompress        # resolves to this package
    from LCT.components.sparse_utils import SparseMuon

Every module of the reference's public surface that has a counterpart here is aliased
(``LCT.operations``, ``LCT.comp_format``, ``LCT.comp_tensor``, ``LCT.tensor_buffer``,
``LCT.LCTensor``, ``LCT.config``, ``LCT.codec.*``, ``LCT.compression.*``, ``LCT.kernels.dispatch``,
``LCT.kernels.backends``, ``LCT.components.{dist_configs,sparse_utils}``).  Nothing is copied: the
aliases are the same module objects, so settings such as ``LCT.config.lane_mapping`` act on
this library.
"""
from __future__ import annotations

import importlib
import sys

_PACKAGE = __name__.rsplit(".", 1)[0]

ALIASED = (
    "", "operations", "comp_format", "comp_tensor", "tensor_buffer", "LCTensor", "config",
    "codec", "codec.encode", "codec.decode", "codec.pointwise", "codec.geometry",
    "compression", "compression.huffman_tables", "compression.probabilities",
    "kernels", "kernels.dispatch", "kernels.backends",
    "components", "components.dist_configs", "components.sparse_utils",
)


def install_as_lct(name: str = "LCT", *, replace: bool = False) -> list[str]:
    """Register the aliases in ``sys.modules``; returns the names installed.  Refuses to shadow
    an already imported package of that name unless ``replace`` is given."""
    if name in sys.modules and not replace:
        existing = sys.modules[name]
        if getattr(existing, "__name__", None) != _PACKAGE:
            raise ImportError(f"a different package is already imported as {name!r}")
    installed = []
    for suffix in ALIASED:
        module = importlib.import_module(_PACKAGE + ("." + suffix if suffix else ""))
        alias = name + ("." + suffix if suffix else "")
        sys.modules[alias] = module
        installed.append(alias)
    return installed
