"""``x @ w.T`` for a quantized ``w``, picking the best available route.

Mirror of src/gguf_jax/_matmul.py.  Three routes, chosen by :func:`matmul`:

- a **fused kernel** (``ggq_gemv`` / ``ggq_gemm``), which keeps the weight quantized in
  HBM and never materializes it;
- **dequantize-then-matmul**, which materializes the whole weight with the decode kernel
  and multiplies with a library GEMM;
- the same thing **split across output rows**, when the whole weight is too large to
  materialize at once.

Both entry points are differentiable in ``x`` through one custom backward, whichever
route the forward took: the backward decodes the weight again (``dx = g @ w``) in the
same row blocks, so the only thing kept for it is the quantized payload.  No gradient
flows to ``w``.
"""
from __future__ import annotations

import functools
import os
from typing import Callable

import numpy as np
import torch
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

from . import _lib, kernels
from .array import QuantizedArray

__all__ = ["dequant_matmul", "fused_batch_limit", "fused_types", "matmul"]

# How large a temporary a single dequantize may allocate before it is split across output
# rows, sized as 4*N*K like the reference (src/gguf_jax/_matmul.py:39-44).
DEQUANT_BLOCK_BYTES = int(os.environ.get("GGUF_JAX_DEQUANT_BLOCK_BYTES", 512 << 20))

FusedEntry = tuple[Callable[..., torch.Tensor], Callable[[QuantizedArray], int]]


@functools.cache
def _fused() -> dict[QT, FusedEntry]:
    """qtype -> (kernel, batch cap for a given weight), asked of the compiled library
    (stands for src/gguf_jax/_matmul.py:52-75).  Raises if the library is not built."""
    L = _lib.lib()
    table: dict[QT, FusedEntry] = {}
    for qt in QT:
        if qt in GGML_QUANT_SIZES and L.ggq_has_fused(int(qt)):
            def cap(w: QuantizedArray, _qt=qt) -> int:
                return int(L.ggq_fused_batch_limit(int(_qt), w.shape[0], w.shape[1]))
            table[qt] = (kernels.fused_matmul, cap)
    return table


def fused_types() -> list[QT]:
    """The qtypes with a fused kernel in this installation."""
    return sorted(_fused().keys(), key=lambda t: t.name)


def fused_batch_limit(w: QuantizedArray) -> int:
    """Largest batch ``w`` can be multiplied at without materializing it; zero when no
    fused kernel applies.  :func:`matmul` consults it for you."""
    entry = _fused().get(w.qtype)
    return entry[1](w) if entry is not None and len(w.shape) == 2 else 0


def matmul(x: torch.Tensor, w: QuantizedArray, *, block_bytes: int | None = None,
           force_fused: bool = False) -> torch.Tensor:
    """``x @ w.T`` with ``w`` quantized, by whichever route fits
    (same contract as src/gguf_jax/_matmul.py:93-125).

    ``x`` is ``(..., K)`` and the result is ``(..., N)`` for ``w`` of shape ``(N, K)``. A
    fused kernel is used when one exists for the qtype, ``x`` is bfloat16, and the
    flattened batch is within that kernel's range; otherwise the weight is dequantized, in
    row blocks if it is too large to do at once.  ``force_fused`` ignores the batch cap.
    """
    if not isinstance(w, QuantizedArray):
        raise TypeError(f"expected a QuantizedArray weight, got {type(w).__name__}")
    if len(w.shape) != 2:
        raise ValueError(f"w must be 2D, got shape {w.shape}")
    if x.shape[-1] != w.shape[1]:
        raise ValueError(
            f"contraction mismatch: x has {x.shape[-1]}, w has {w.shape[1]}")

    kernel = None
    entry = _fused().get(w.qtype)
    if entry is not None and x.dtype == torch.bfloat16:
        batch = int(np.prod(x.shape[:-1], dtype=np.int64))
        if force_fused or batch <= entry[1](w):
            kernel = entry[0]
    return _frozen_matmul(x, w, kernel, _blocks(w, block_bytes))


def dequant_matmul(x: torch.Tensor, w: QuantizedArray, *, block_bytes: int | None = None) -> torch.Tensor:
    """``x @ w.T`` by materializing ``w`` (in row blocks when it is large), never more than
    ``block_bytes`` of dense weight at a time (src/gguf_jax/_matmul.py:128-162)."""
    if not isinstance(w, QuantizedArray):
        raise TypeError(f"expected a QuantizedArray weight, got {type(w).__name__}")
    return _frozen_matmul(x, w, None, _blocks(w, block_bytes))


def _blocks(w: QuantizedArray, block_bytes: int | None) -> int:
    return _block_count(*w.shape, DEQUANT_BLOCK_BYTES if block_bytes is None else block_bytes)


class _FrozenMatmul(torch.autograd.Function):
    """Forward by ``kernel`` or by dequantizing in ``blocks``; backward ``dx = g @ w`` with
    only the quantized payload saved (src/gguf_jax/_matmul.py:170-192)."""

    @staticmethod
    def forward(ctx, x, data, qtype, shape, dtype, kernel, blocks):
        w = QuantizedArray(data=data, qtype=qtype, shape=shape, dtype=dtype)
        ctx.save_for_backward(data)
        ctx.meta = (qtype, shape, dtype, blocks, x.dtype)
        if kernel is not None:
            return kernel(x, w)
        return _dequant_forward(x, w, blocks)

    @staticmethod
    def backward(ctx, g):
        (data,) = ctx.saved_tensors
        qtype, shape, dtype, blocks, x_dtype = ctx.meta
        w = QuantizedArray(data=data, qtype=qtype, shape=shape, dtype=dtype)
        return _dequant_backward(g, w, blocks).to(x_dtype), None, None, None, None, None, None


def _frozen_matmul(x, w: QuantizedArray, kernel, blocks: int) -> torch.Tensor:
    if torch.is_grad_enabled() and x.requires_grad:
        return _FrozenMatmul.apply(x, w.data, w.qtype, w.shape, w.dtype, kernel, blocks)
    if kernel is not None:
        return kernel(x, w)
    return _dequant_forward(x, w, blocks)


def _mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` with numpy-style dtype promotion (an f16 ``x`` against a bf16 weight
    promotes to f32, as in the reference)."""
    dt = torch.promote_types(a.dtype, b.dtype)
    return torch.matmul(a.to(dt), b.to(dt))


def _dequant_forward(x: torch.Tensor, w: QuantizedArray, blocks: int) -> torch.Tensor:
    out_rows, in_features = w.shape
    if blocks == 1:
        return _mm(x, w.dequantize().T)
    rows = out_rows // blocks
    flat = x.reshape(-1, in_features)
    data = w.data.reshape(blocks, rows, -1)
    out = None
    for i in range(blocks):
        sub = QuantizedArray(data=data[i], qtype=w.qtype, shape=(rows, in_features), dtype=w.dtype)
        part = _mm(flat, sub.dequantize().T)
        if out is None:
            out = torch.empty((flat.shape[0], out_rows), dtype=part.dtype, device=part.device)
        out[:, i * rows:(i + 1) * rows] = part
    return out.reshape(*x.shape[:-1], out_rows)


def _dequant_backward(g: torch.Tensor, w: QuantizedArray, blocks: int) -> torch.Tensor:
    """``g @ w``, the cotangent of ``x``, decoding ``w`` as the forward did; row blocks
    partition the contraction, so their products are summed in float32."""
    out_rows, in_features = w.shape
    if blocks == 1:
        return _mm(g, w.dequantize())
    rows = out_rows // blocks
    flat = g.reshape(-1, out_rows)
    data = w.data.reshape(blocks, rows, -1)
    acc = torch.zeros((flat.shape[0], in_features), dtype=torch.float32, device=g.device)
    for i in range(blocks):
        sub = QuantizedArray(data=data[i], qtype=w.qtype, shape=(rows, in_features), dtype=w.dtype)
        acc += _mm(flat[:, i * rows:(i + 1) * rows], sub.dequantize()).float()
    return acc.reshape(*g.shape[:-1], in_features)


def _block_count(out_rows: int, in_features: int, budget: int) -> int:
    """How many row blocks keep one dequantize under ``budget``; constrained to divisors
    of ``out_rows`` so the blocks are uniform (src/gguf_jax/_matmul.py:247-260)."""
    needed = 4 * out_rows * in_features
    if needed <= budget:
        return 1
    target = -(-needed // budget)
    for n in range(target, out_rows + 1):
        if out_rows % n == 0:
            return n
    return out_rows
