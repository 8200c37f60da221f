"""QuantizedArray: a pytree holding a GGUF-quantized tensor on the device.

Mirror of src/gguf_jax/array.py with torch tensors as the array type: same fields, same
methods, same errors.  The uint8 payload layout ``(*shape[:-1], row_bytes)`` is the ABI
the CUDA kernels read directly.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any

import numpy as np
import torch
from gguf.constants import GGML_QUANT_SIZES, GGMLQuantizationType
from torch.utils import _pytree

from . import _backend, quants

__all__ = ["QuantizedArray", "quantize"]

# Types kept as native (non-uint8) arrays: dequantize is a cast (or identity).
_NATIVE_TYPES = {
    GGMLQuantizationType.I8: torch.int8,
    GGMLQuantizationType.I16: torch.int16,
    GGMLQuantizationType.I32: torch.int32,
    GGMLQuantizationType.I64: torch.int64,
    GGMLQuantizationType.F64: torch.float64,
}

_INTEGER_TYPES = {
    GGMLQuantizationType.I8,
    GGMLQuantizationType.I16,
    GGMLQuantizationType.I32,
    GGMLQuantizationType.I64,
}


@dataclass
class QuantizedArray:
    """A quantized tensor: raw GGUF block data plus the metadata to decode it.

    ``data`` is the payload as stored in the GGUF file: a uint8 tensor of shape
    ``(*shape[:-1], row_bytes)`` for quantized/float qtypes (F16/F32/BF16 included), or a
    native integer/float tensor for the plain I8/I16/I32/I64/F64 types.

    It is a pytree with exactly one leaf (``data``); ``qtype``, ``shape`` and ``dtype`` are
    static metadata (src/gguf_jax/array.py:33-50).
    """

    data: torch.Tensor
    qtype: GGMLQuantizationType = field(metadata={"static": True})
    shape: tuple[int, ...] = field(metadata={"static": True})
    dtype: Any = field(default=torch.bfloat16, metadata={"static": True})

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    @property
    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    @property
    def device(self) -> torch.device:
        return self.data.device

    def to(self, device) -> "QuantizedArray":
        """Same array with the payload moved to ``device``."""
        return replace(self, data=self.data.to(device))

    def astype(self, dtype) -> "QuantizedArray":
        """Return a copy whose default dequantization dtype is ``dtype``."""
        return replace(self, dtype=_backend.canon_dtype(dtype))

    def dequantize(self, dtype=None) -> torch.Tensor:
        """Decode to a dense tensor of ``dtype`` (default: ``self.dtype``).

        Decoding computes in float32, bitwise identical to ``gguf.quants.dequantize``, and
        rounds once to ``dtype`` inside the kernel. Integer qtypes are returned as-is.
        """
        dtype = self.dtype if dtype is None else _backend.canon_dtype(dtype)
        if self.qtype in _NATIVE_TYPES:
            out = self.data.reshape(self.shape)
            if self.qtype in _INTEGER_TYPES:
                return out
            return out.to(dtype)
        return quants.dequantize(self.data, self.qtype, dtype).reshape(self.shape)

    def __repr__(self) -> str:
        name = str(self.dtype).replace("torch.", "")
        return f"QuantizedArray({self.qtype.name}, shape={self.shape}, dtype={name})"

    @classmethod
    def from_bytes(cls, data, qtype: GGMLQuantizationType, shape: tuple[int, ...] | None = None,
                   dtype=torch.bfloat16, device=None) -> "QuantizedArray":
        """Wrap raw quantized bytes (numpy or torch uint8, byte-shaped) as a QuantizedArray
        (src/gguf_jax/array.py:87-104)."""
        data = _backend.as_tensor(data, device)
        dtype = _backend.canon_dtype(dtype)
        if qtype in _NATIVE_TYPES:
            shape = tuple(data.shape) if shape is None else tuple(shape)
            return cls(data=data.reshape(shape), qtype=qtype, shape=shape, dtype=dtype)
        if data.dtype != torch.uint8:
            raise ValueError(f"expected uint8 data for {qtype.name}, got {data.dtype}")
        if shape is None:
            shape = quants._ref.quant_shape_from_byte_shape(tuple(data.shape), qtype)
        shape = tuple(int(s) for s in shape)
        block_size, type_size = GGML_QUANT_SIZES[qtype]
        expected = shape[-1] // block_size * type_size
        data = data.reshape(*shape[:-1], expected)
        return cls(data=data, qtype=qtype, shape=shape, dtype=dtype)


def _flatten(a: QuantizedArray):
    return [a.data], (a.qtype, a.shape, a.dtype)


def _unflatten(leaves, ctx):
    return QuantizedArray(leaves[0], *ctx)


_pytree.register_pytree_node(
    QuantizedArray, _flatten, _unflatten,
    serialized_type_name="gguf_jax_b200.QuantizedArray")


def quantize(array, qtype: GGMLQuantizationType, dtype=torch.bfloat16, device=None) -> QuantizedArray:
    """Quantize an array on the host through gguf-py (src/gguf_jax/array.py:107-119).

    Only the qtypes gguf-py can quantize are supported; a convenience for tests and tools.
    """
    import gguf

    if isinstance(array, torch.Tensor):
        array = array.detach().to("cpu", torch.float32).numpy()
    np_arr = np.asarray(array, dtype=np.float32)
    qdata = gguf.quants.quantize(np_arr, qtype)
    if qdata.dtype != np.uint8:
        qdata = np.ascontiguousarray(qdata).view(np.uint8)
    return QuantizedArray.from_bytes(qdata, qtype, shape=np_arr.shape, dtype=dtype, device=device)
