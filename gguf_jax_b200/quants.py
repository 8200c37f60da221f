"""Block dequantization for GGUF/GGML quantized tensor formats on B200.

Host-side mirror of the reference's ``quants`` module (src/gguf_jax/quants.py): the same
registry (``register_dequant``, ``supported_types``), the same entry points
(``dequantize_blocks``, ``dequantize``) and the same errors, with every built-in decoder
backed by the CUDA decode kernel behind ``ggq_dequant`` (include/ggq.h).  The float32
output is bitwise identical to ``gguf.quants.dequantize``; other dtypes are that result
rounded once, inside the kernel.

Layout convention (same as gguf-py and the reference): a quantized tensor is uint8 bytes
of shape ``(..., row_bytes)`` whose last axis packs ``row_bytes // type_size`` blocks of
``block_size`` elements.
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
from gguf import quants as _ref
from gguf.constants import GGML_QUANT_SIZES, GGMLQuantizationType

from . import _backend, _lib

__all__ = [
    "GGMLQuantizationType",
    "dequantize",
    "dequantize_blocks",
    "register_dequant",
    "supported_types",
]

# fn(blocks: uint8[n_blocks, type_size], dtype) -> dtype[n_blocks, block_size]
# The result must equal the bitwise-exact float32 decode rounded once to ``dtype``.
DequantFn = Callable[[torch.Tensor, Any], torch.Tensor]

_DEQUANT: dict[GGMLQuantizationType, DequantFn] = {}


def register_dequant(qtype: GGMLQuantizationType, fn: DequantFn, *, override: bool = False) -> None:
    """Register a block-dequantization kernel for ``qtype``
    (same contract as src/gguf_jax/quants.py:44-56).

    ``fn`` maps ``uint8[n_blocks, type_size]`` plus a target dtype to
    ``dtype[n_blocks, block_size]``. Pass ``override=True`` to replace a built-in kernel.
    """
    if qtype in _DEQUANT and not override:
        raise ValueError(f"dequant kernel for {qtype.name} already registered")
    _DEQUANT[qtype] = fn


def supported_types() -> list[GGMLQuantizationType]:
    return sorted(_DEQUANT.keys(), key=lambda t: t.name)


def _builtin(qtype: GGMLQuantizationType) -> DequantFn:
    block_size, type_size = GGML_QUANT_SIZES[qtype]

    def kernel(blocks: torch.Tensor, dtype) -> torch.Tensor:
        dtype = _backend.canon_dtype(dtype)
        dev = _backend.require_cuda(blocks, f"dequantize({qtype.name})")
        _lib.ensure_tables(dev)
        blocks = blocks.contiguous()
        n_blocks = blocks.shape[0]
        out = torch.empty((n_blocks, block_size), dtype=dtype, device=blocks.device)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().ggq_dequant(
                int(qtype), blocks.data_ptr(), n_blocks, out.data_ptr(),
                _backend.dtype_code(dtype), _backend.stream_ptr(dev)))
        return out

    kernel.__name__ = f"dequant_{qtype.name.lower()}"
    return kernel


# The decodable set is gguf-py's own (quants._type_traits) plus the two float
# passthroughs it special-cases, as in the reference (tests/test_bitwise.py:104-110).
for _qt in (*_ref._type_traits.keys(), GGMLQuantizationType.F16, GGMLQuantizationType.F32):
    if _qt not in _DEQUANT:
        register_dequant(_qt, _builtin(_qt))


def dequantize_blocks(blocks: torch.Tensor, qtype: GGMLQuantizationType, dtype=torch.float32) -> torch.Tensor:
    """Dequantize ``uint8[n_blocks, type_size]`` to ``dtype[n_blocks, block_size]``
    (src/gguf_jax/quants.py:718-730)."""
    block_size, type_size = GGML_QUANT_SIZES[qtype]
    if qtype not in _DEQUANT:
        raise NotImplementedError(f"Dequantization for {qtype.name} is not implemented")
    blocks = _backend.as_tensor(blocks)
    if blocks.dtype != torch.uint8 or blocks.ndim != 2 or blocks.shape[-1] != type_size:
        raise ValueError(
            f"expected uint8 blocks of shape (n_blocks, {type_size}) for {qtype.name}, "
            f"got {blocks.dtype} {tuple(blocks.shape)}")
    out = _DEQUANT[qtype](blocks, dtype)
    assert tuple(out.shape) == (blocks.shape[0], block_size)
    return out


def dequantize(data, qtype: GGMLQuantizationType, dtype=torch.float32) -> torch.Tensor:
    """Dequantize a byte-shaped uint8 array ``(..., row_bytes)`` to
    ``(..., row_bytes // type_size * block_size)`` (src/gguf_jax/quants.py:733-745).

    With ``dtype=float32`` the result is bitwise identical to ``gguf.quants.dequantize``;
    other dtypes are that result rounded once.
    """
    _, type_size = GGML_QUANT_SIZES[qtype]
    data = _backend.as_tensor(data)
    shape = _ref.quant_shape_from_byte_shape(tuple(data.shape), qtype)  # raises ValueError on a bad row size
    blocks = data.reshape(-1, type_size)
    return dequantize_blocks(blocks, qtype, dtype).reshape(shape)
