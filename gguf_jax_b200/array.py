"""QuantizedArray: GGUF block bytes on the device plus what is needed to decode them.

Public contract of the reference's container (src/gguf_jax/array.py:33-119): the fields
``data / qtype / shape / dtype``, the properties ``ndim / size / nbytes``, ``astype``,
``dequantize``, ``from_bytes`` and the module-level ``quantize``, with the same errors.
Here the array type is a torch tensor and the payload layout ``uint8[*shape[:-1], row_bytes]``
is exactly what the CUDA kernels index, so a row range of a 2-D weight is a byte slice.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any

import numpy as np
import torch
from gguf.constants import GGML_QUANT_SIZES, GGMLQuantizationType
from torch.utils import _pytree

from . import _backend, quants

__all__ = ["QuantizedArray", "quantize"]

_QT = GGMLQuantizationType
# GGUF also stores plain integer / float64 tensors.  They are held in their own element type
# instead of as bytes; the flag says whether "dequantize" leaves them alone (integers) or casts.
_PLAIN: dict[GGMLQuantizationType, tuple[torch.dtype, bool]] = {
    _QT.I8: (torch.int8, True), _QT.I16: (torch.int16, True), _QT.I32: (torch.int32, True),
    _QT.I64: (torch.int64, True), _QT.F64: (torch.float64, False),
}
# Used by the loader to decide whether a tensor's bytes need a uint8 view.
_NATIVE_TYPES = {qt: spec[0] for qt, spec in _PLAIN.items()}


def _row_bytes(qtype: GGMLQuantizationType, n_cols: int) -> int:
    per_block, block_bytes = GGML_QUANT_SIZES[qtype]
    return n_cols // per_block * block_bytes


@dataclasses.dataclass
class QuantizedArray:
    """One tensor of a GGUF file, still in its storage format.

    ``data``   the only tensor inside (and the only pytree leaf): ``uint8[*shape[:-1], row_bytes]``
               for every block format and for F16/F32/BF16, or an int8/16/32/64 / float64 tensor
               of ``shape`` for the plain GGUF element types;
    ``qtype``  the GGML storage format;
    ``shape``  logical shape after decoding;
    ``dtype``  what :meth:`dequantize` returns when not told otherwise.
    The last three are static metadata: tree maps see one leaf and carry them along.
    """

    data: torch.Tensor
    qtype: GGMLQuantizationType = dataclasses.field(metadata={"static": True})
    shape: tuple[int, ...] = dataclasses.field(metadata={"static": True})
    dtype: Any = dataclasses.field(default=torch.bfloat16, metadata={"static": True})

    # ---- shape-like properties of the logical tensor
    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return math.prod(self.shape)

    @property
    def nbytes(self) -> int:
        """Bytes held in device memory (the quantized payload, not the decoded size)."""
        return self.data.element_size() * self.data.numel()

    @property
    def device(self) -> torch.device:
        return self.data.device

    def __repr__(self) -> str:
        return f"QuantizedArray({self.qtype.name}, shape={self.shape}, dtype={str(self.dtype).removeprefix('torch.')})"

    # ---- cheap views
    def to(self, device) -> "QuantizedArray":
        """The same tensor with its payload on ``device``."""
        return dataclasses.replace(self, data=self.data.to(device))

    def astype(self, dtype) -> "QuantizedArray":
        """Same payload, different default output dtype for :meth:`dequantize`."""
        return dataclasses.replace(self, dtype=_backend.canon_dtype(dtype))

    # ---- decoding
    def dequantize(self, dtype=None) -> torch.Tensor:
        """Dense tensor of ``shape``.  Block formats go through the CUDA decode kernel: float32
        arithmetic bit-identical to ``gguf.quants.dequantize``, rounded once to the requested
        dtype inside the kernel.  Plain integer tensors come back unchanged, float64 is cast."""
        want = self.dtype if dtype is None else _backend.canon_dtype(dtype)
        plain = _PLAIN.get(self.qtype)
        if plain is None:
            return quants.dequantize(self.data, self.qtype, want).reshape(self.shape)
        dense = self.data.reshape(self.shape)
        return dense if plain[1] else dense.to(want)

    # ---- construction
    @classmethod
    def from_bytes(cls, data, qtype: GGMLQuantizationType, shape: tuple[int, ...] | None = None,
                   dtype=torch.bfloat16, device=None) -> "QuantizedArray":
        """Wrap a payload (numpy array, torch tensor or buffer) without touching its bytes.

        For block formats ``data`` must be uint8 (``ValueError`` otherwise) shaped
        ``(..., row_bytes)``; ``shape`` defaults to what that byte shape implies
        (``row_bytes / block_bytes * block_elems`` columns) and, when given, the payload is
        reshaped to match it.  Plain integer / float64 tensors keep their element type.
        """
        payload = _backend.as_tensor(data, device)
        out_dtype = _backend.canon_dtype(dtype)
        if qtype in _PLAIN:
            logical = tuple(payload.shape) if shape is None else tuple(int(s) for s in shape)
            return cls(payload.reshape(logical), qtype, logical, out_dtype)
        if payload.dtype != torch.uint8:
            raise ValueError(f"expected uint8 data for {qtype.name}, got {payload.dtype}")
        if shape is None:
            logical = tuple(quants._ref.quant_shape_from_byte_shape(tuple(payload.shape), qtype))
        else:
            logical = tuple(int(s) for s in shape)
        payload = payload.reshape(*logical[:-1], _row_bytes(qtype, logical[-1]))
        return cls(payload, qtype, logical, out_dtype)


_pytree.register_pytree_node(
    QuantizedArray,
    lambda qa: ([qa.data], (qa.qtype, qa.shape, qa.dtype)),
    lambda leaves, meta: QuantizedArray(leaves[0], *meta),
    serialized_type_name="gguf_jax_b200.QuantizedArray")


def quantize(array, qtype: GGMLQuantizationType, dtype=torch.bfloat16, device=None) -> QuantizedArray:
    """Host-side quantization through gguf-py, for the formats gguf-py can encode
    (src/gguf_jax/array.py:107-119); meant for tests and small tools, not for a hot path."""
    import gguf

    if isinstance(array, torch.Tensor):
        array = array.detach().cpu().float().numpy()
    dense = np.asarray(array, dtype=np.float32)
    packed = np.ascontiguousarray(gguf.quants.quantize(dense, qtype))
    if packed.dtype != np.uint8:
        packed = packed.view(np.uint8)
    return QuantizedArray.from_bytes(packed, qtype, shape=dense.shape, dtype=dtype, device=device)
