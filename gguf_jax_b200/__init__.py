"""gguf_jax_b200: GGUF-quantized tensors on B200, dequantized on the fly by CUDA kernels.

Drop-in for the public surface of gguf-jax (src/gguf_jax/__init__.py:15-29) with torch
tensors as the array type.  Quantized tensors stay as raw uint8 block data in
:class:`QuantizedArray` pytrees; decoding and the fused multiplies run in hand-written
sm_100a kernels behind the C ABI of include/ggq.h.  The float32 decode is bitwise
identical to ``gguf.quants``.
"""

from gguf.constants import GGMLQuantizationType

from .array import QuantizedArray, quantize
from .loader import GGUFFile, load_gguf
from ._matmul import dequant_matmul, fused_batch_limit, fused_types, matmul
from .quants import dequantize, dequantize_blocks, register_dequant, supported_types

__all__ = [
    "GGMLQuantizationType",
    "GGUFFile",
    "QuantizedArray",
    "dequant_matmul",
    "dequantize",
    "dequantize_blocks",
    "fused_batch_limit",
    "fused_types",
    "load_gguf",
    "matmul",
    "quantize",
    "register_dequant",
    "supported_types",
]
