"""B200-native lossless BF16 tensor codec with the LCT Python API.

Sub-modules mirror the reference's module paths (``operations``, ``comp_format``,
``comp_tensor``, ``tensor_buffer``, ``LCTensor``, ``codec.*``, ``compression.*``,
``kernels.dispatch``).  Nothing heavy is imported here; the CUDA library is
loaded on first use by ``kernels.dispatch``.
"""

__all__ = [
    "comp_format", "comp_tensor", "tensor_buffer", "operations", "LCTensor",
    "codec", "compression", "kernels", "config", "sharded", "serialization",
]
