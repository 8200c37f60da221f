"""Router for ``x @ w.T`` with a quantized ``w``.

Public contract of the reference's router (src/gguf_jax/_matmul.py:52-260): ``matmul``,
``dequant_matmul``, ``fused_types``, ``fused_batch_limit``; same argument meaning, same errors,
gradient in ``x`` only.  What is behind them is this library's own:

* **fused** -- one launch of the CUDA kernels over the quantized bytes.  Which kernel
  (small-batch GEMV, or the tcgen05 GEMM above it) and up to which batch is decided by the
  compiled library (``ggq_fused_batch_limit``), per qtype and shape; this module only asks.
* **materialize** -- the decode kernel writes a dense bf16/f32 copy of ``w`` (all of it, or
  ``R`` equal row slabs when the copy would exceed a byte budget) and a library GEMM multiplies.

The backward pass is the same for both: ``dx = g @ w`` with ``w`` decoded again slab by slab,
so only the quantized payload is kept alive between forward and backward.
"""
from __future__ import annotations

import functools
import math
import os
from typing import Callable

import torch
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

from . import _backend, _lib, kernels
from .array import QuantizedArray

__all__ = ["dequant_matmul", "fused_batch_limit", "fused_types", "matmul"]

# Byte budget of one dense slab.  The reference's environment knob and default are kept
# (src/gguf_jax/_matmul.py:39-44); like there, a slab is costed at 4 bytes per weight.
DEQUANT_BLOCK_BYTES = int(os.environ.get("GGUF_JAX_DEQUANT_BLOCK_BYTES", 512 << 20))

FusedEntry = tuple[Callable[..., torch.Tensor], Callable[[QuantizedArray], int]]


@functools.cache
def _fused() -> dict[QT, FusedEntry]:
    """``qtype -> (kernel, cap(w))`` for every qtype the compiled library multiplies fused.
    Loading the library is the only way to know, so a missing build raises here."""
    L = _lib.lib()

    def entry(qt: QT) -> FusedEntry:
        code = int(qt)
        caps: dict[tuple[int, int], int] = {}       # the library's answer depends on the shape only

        def cap(w) -> int:
            got = caps.get(w.shape)
            if got is None:
                got = caps[w.shape] = int(L.ggq_fused_batch_limit(code, w.shape[0], w.shape[1]))
            return got

        return kernels.fused_matmul, cap

    return {qt: entry(qt) for qt in QT if qt in GGML_QUANT_SIZES and L.ggq_has_fused(int(qt))}


def fused_types() -> list[QT]:
    """Qtypes that have a fused kernel, sorted by name."""
    return sorted(_fused(), key=lambda qt: qt.name)


def fused_batch_limit(w: QuantizedArray) -> int:
    """Largest flattened batch at which :func:`matmul` still multiplies ``w`` without
    materializing it (0: never)."""
    hit = _fused().get(w.qtype)
    return hit[1](w) if hit is not None and len(w.shape) == 2 else 0


def _validate(x: torch.Tensor, w) -> None:
    if not isinstance(w, QuantizedArray):
        raise TypeError(f"expected a QuantizedArray weight, got {type(w).__name__}")
    if len(w.shape) != 2:
        raise ValueError(f"w must be 2D, got shape {w.shape}")
    if x.shape[-1] != w.shape[1]:
        raise ValueError(f"contraction mismatch: x has {x.shape[-1]}, w has {w.shape[1]}")


def matmul(x: torch.Tensor, w: QuantizedArray, *, block_bytes: int | None = None,
           force_fused: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x (..., K) @ w(N, K).T -> (..., N)``.

    Fused when ``w.qtype`` has a kernel, ``x`` is bfloat16 and the flattened batch does not
    exceed :func:`fused_batch_limit`; ``force_fused=True`` skips the batch test (the kernels
    accept any batch; beyond the limit they are merely slower than materializing).  Everything
    else is materialized under the ``block_bytes`` budget (default
    :data:`DEQUANT_BLOCK_BYTES`).  ``TypeError`` for a weight that is not a
    :class:`QuantizedArray`, ``ValueError`` for a weight that is not 2-D or a contraction mismatch.

    Host-resident operands (an extension; the reference's arrays are device arrays): ``x`` may be a
    pinned CPU tensor and ``out`` a pinned CPU (or device) tensor of the result's shape.  They are
    served by the fused route only (see :func:`gguf_jax_b200.kernels.fused_matmul`), without
    gradients; anything the fused route does not take raises ``ValueError``.
    """
    _validate(x, w)
    route = None
    hit = _fused().get(w.qtype)
    if hit is not None and x.dtype == torch.bfloat16:
        batch = math.prod(x.shape[:-1])
        if force_fused or batch <= hit[1](w):
            route = hit[0]
    if out is not None or not x.is_cuda:
        _backend.require_cuda(w.data, "matmul")
        if route is None:
            raise ValueError("host-resident activations and caller-owned results are served by the fused kernels only "
                             f"(bfloat16 x, a fused qtype, batch within fused_batch_limit); got {w.qtype.name}, {x.dtype}, "
                             f"batch {math.prod(x.shape[:-1])}")
        return route(x, w, out=out)
    return _apply(x, w, route, _slab_count(w, block_bytes))


def dequant_matmul(x: torch.Tensor, w: QuantizedArray, *, block_bytes: int | None = None) -> torch.Tensor:
    """The materializing route on its own: decode ``w`` (in row slabs of at most ``block_bytes``
    when it is large) and multiply with a library GEMM.  The result dtype is the promotion of
    ``x.dtype`` and ``w.dtype``."""
    if not isinstance(w, QuantizedArray):
        raise TypeError(f"expected a QuantizedArray weight, got {type(w).__name__}")
    return _apply(x, w, None, _slab_count(w, block_bytes))


# ---------------------------------------------------------------------------------------------
# slabs

def _block_count(out_rows: int, in_features: int, budget: int) -> int:
    """Number of equal row slabs so that one slab, costed at 4 bytes per weight, fits ``budget``:
    the smallest divisor of ``out_rows`` that is large enough (``out_rows`` itself if none is)."""
    slabs_wanted = max(1, math.ceil(4 * out_rows * in_features / max(budget, 1)))
    return next((d for d in range(slabs_wanted, out_rows) if out_rows % d == 0), out_rows) if slabs_wanted > 1 else 1


def _slab_count(w: QuantizedArray, block_bytes: int | None) -> int:
    return _block_count(w.shape[0], w.shape[1], DEQUANT_BLOCK_BYTES if block_bytes is None else block_bytes)


def _slabs(w: QuantizedArray, count: int):
    """``(first_row, dense slab)`` for each of ``count`` equal row slabs, decoded one at a time."""
    rows = w.shape[0] // count
    for i in range(count):
        part = QuantizedArray(w.data[i * rows:(i + 1) * rows], w.qtype, (rows, w.shape[1]), w.dtype)
        yield i * rows, part.dequantize()


def _promoted_mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    common = torch.promote_types(a.dtype, b.dtype)
    return torch.matmul(a.to(common), b.to(common))


def _materialized_forward(x: torch.Tensor, w: QuantizedArray, count: int) -> torch.Tensor:
    n_out = w.shape[0]
    x2 = x.reshape(-1, w.shape[1])
    y = None
    for row0, dense in _slabs(w, count):
        part = _promoted_mm(x2, dense.T)
        if count == 1:
            y = part
            break
        if y is None:
            y = part.new_empty((x2.shape[0], n_out))
        y[:, row0:row0 + dense.shape[0]] = part
    return y.reshape(*x.shape[:-1], n_out)


def _input_cotangent(g: torch.Tensor, w: QuantizedArray, count: int) -> torch.Tensor:
    """``g (..., N) @ w (N, K)``: the slabs cut the contraction, so their products add up (in
    float32 when there is more than one)."""
    g2 = g.reshape(-1, w.shape[0])
    if count == 1:
        (_, dense), = _slabs(w, 1)
        return _promoted_mm(g2, dense).reshape(*g.shape[:-1], w.shape[1])
    total = torch.zeros((g2.shape[0], w.shape[1]), dtype=torch.float32, device=g.device)
    for row0, dense in _slabs(w, count):
        total += _promoted_mm(g2[:, row0:row0 + dense.shape[0]], dense).float()
    return total.reshape(*g.shape[:-1], w.shape[1])


# ---------------------------------------------------------------------------------------------
# one differentiable wrapper around whichever forward was chosen

class _QuantizedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, payload, meta, route, count):
        ctx.save_for_backward(payload)
        ctx.extra = (meta, count, x.dtype)
        w = QuantizedArray(payload, *meta)
        return route(x, w) if route is not None else _materialized_forward(x, w, count)

    @staticmethod
    def backward(ctx, g):
        (payload,) = ctx.saved_tensors
        meta, count, x_dtype = ctx.extra
        dx = _input_cotangent(g, QuantizedArray(payload, *meta), count).to(x_dtype)
        return dx, None, None, None, None


def _apply(x: torch.Tensor, w: QuantizedArray, route, count: int) -> torch.Tensor:
    if x.requires_grad and torch.is_grad_enabled():
        return _QuantizedLinear.apply(x, w.data, (w.qtype, w.shape, w.dtype), route, count)
    return route(x, w) if route is not None else _materialized_forward(x, w, count)
