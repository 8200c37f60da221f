"""Fused multiply kernels: ``x @ w.T`` with ``w`` kept quantized in HBM.

Host-side wrappers over ``ggq_gemv`` / ``ggq_gemm`` (include/ggq.h).  They stand where the
reference's ``matmul_q4_k``, ``matmul_q5_k``, ``matmul_q6_k``, ``matmul_iq4_xs``,
``matmul_lowbit`` and ``gemm_q4_k`` stand (src/gguf_jax/cute/*.py) and keep their
calling convention: ``x`` is bfloat16 ``(..., K)``, ``w`` a 2-D ``QuantizedArray (N, K)``,
the result is bfloat16 ``(..., N)``.

Numerical contract: weights enter at full float32 precision (integer codes times float32
scales), accumulation is float32 and the only narrow rounding is the output, so the
result tracks the float32 ``dequant_matmul`` within relative L2 2e-3 and a one-hot ``x``
reproduces ``bf16(float32 weight)`` exactly.
"""
from __future__ import annotations

import torch
from gguf.constants import GGMLQuantizationType as QT

from . import _backend, _lib
from .array import QuantizedArray

__all__ = [
    "LOWBIT_TYPES", "fused_matmul", "gemv_max_batch", "matmul_q4_k", "matmul_q5_k", "matmul_q6_k",
    "matmul_iq4_xs", "matmul_lowbit", "gemm_q4_k", "dequantize_q4_k", "register",
]

# The eight types the reference's low-bit template covers (src/gguf_jax/cute/lowbit.py).
LOWBIT_TYPES = (QT.Q2_K, QT.IQ1_S, QT.IQ1_M, QT.IQ2_XXS, QT.IQ2_XS, QT.IQ2_S, QT.IQ3_XXS, QT.IQ3_S)


_ws_need: dict[tuple[int, int, int, int], int] = {}
_cap: list[int] = []


def _gemv_cap(L) -> int:
    if not _cap:
        _cap.append(int(L.ggq_gemv_max_batch()))
    return _cap[0]


def gemv_max_batch() -> int:
    """Largest flattened batch served by the small-batch kernel (``ggq_gemv``)."""
    return int(_lib.lib().ggq_gemv_max_batch())


def _check(x: torch.Tensor, w: QuantizedArray, qtypes=None) -> tuple[int, int]:
    if not isinstance(w, QuantizedArray):
        raise TypeError(f"expected a QuantizedArray weight, got {type(w).__name__}")
    if qtypes is not None and w.qtype not in qtypes:
        raise ValueError(f"this kernel handles {[t.name for t in qtypes]}, got {w.qtype.name}")
    if len(w.shape) != 2:
        raise ValueError(f"w must be 2D, got shape {w.shape}")
    n_rows, k_dim = w.shape
    if x.shape[-1] != k_dim:
        raise ValueError(f"contraction mismatch: x has {x.shape[-1]}, w has {k_dim}")
    if x.dtype != torch.bfloat16:
        raise ValueError(f"x must be bfloat16, got {x.dtype}")
    return n_rows, k_dim


def fused_matmul(x: torch.Tensor, w: QuantizedArray, *, out_dtype=torch.bfloat16, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T`` through the fused kernels, whatever the batch: ``ggq_gemv`` up to
    ``gemv_max_batch()`` rows (tuned batch-1, tiled, batch-major or small-weight MMA kernel, chosen
    by the library per format, batch and weight size), ``ggq_gemm`` above it (Q4_K / Q5_K / Q6_K:
    the batch-major kernel up to 32 rows, then the bf16-weight tcgen05 kernel; other formats: the
    tf32 tcgen05 kernel).

    Host-resident operands: ``x`` may be a *pinned* CPU tensor (it is brought to the device by
    ``ggq_stage_host``, a small kernel in front of the product, instead of a copy-engine transfer),
    and ``out`` may be a pinned CPU tensor of the result's shape (up to ``gemv_max_batch()`` rows):
    the kernel then stores the result straight into host memory, readable once the stream has been
    synchronised.  Pageable host memory is refused; there is no CPU computation."""
    n_rows, k_dim = _check(x, w)
    dev = _backend.require_cuda(w.data, f"fused matmul ({w.qtype.name})")
    host_x = not x.is_cuda
    if host_x:
        if not x.is_pinned():
            raise RuntimeError("fused matmul: x lives in pageable host memory; pin it (x.pin_memory()) or move it to "
                               "the device - the library computes on the GPU only")
    elif x.device != w.data.device:
        raise ValueError(f"x is on {x.device}, w on {w.data.device}")
    _lib.ensure_tables(dev)
    L = _lib.lib()
    xm = x.reshape(-1, k_dim).contiguous()
    m = xm.shape[0]
    # the common case (the tensors live on the current device) skips the device switch, which
    # costs more host time than the rest of this function
    prev = torch.cuda.current_device()
    if prev != dev:
        torch.cuda.set_device(dev)
    try:
        stream = _backend.stream_ptr(dev)
        x_ptr = xm.data_ptr()
        if host_x and m > 0:
            # first thing, so that the fetch runs on the GPU while the host prepares the product's launch
            nbytes = m * k_dim * 2
            xd = _backend.staging(dev, nbytes, stream)
            _lib.check(L.ggq_stage_host(x_ptr, xd.data_ptr(), nbytes, stream))
            x_ptr = xd.data_ptr()
        data = w.data.contiguous()
        if out is not None:
            if tuple(out.shape) != (*x.shape[:-1], n_rows) or not out.is_contiguous():
                raise ValueError(f"out must be contiguous with shape {(*x.shape[:-1], n_rows)}, got {tuple(out.shape)}")
            if out.is_cuda:
                if out.device != w.data.device:
                    raise ValueError(f"out is on {out.device}, w on {w.data.device}")
            elif not out.is_pinned():
                raise RuntimeError("fused matmul: out lives in pageable host memory; pin it or use a device tensor")
            elif m > _gemv_cap(L):
                raise ValueError(f"a host result buffer is served up to {_gemv_cap(L)} batch rows, got {m}")
            out_dtype = out.dtype
            y = out.view(m, n_rows)
        else:
            out_dtype = _backend.canon_dtype(out_dtype)
            y = torch.empty((m, n_rows), dtype=out_dtype, device=w.data.device)
        if m == 0:
            return y.reshape(*x.shape[:-1], n_rows)
        fn = L.ggq_gemv if m <= _gemv_cap(L) else L.ggq_gemm
        key = (int(w.qtype), n_rows, k_dim, m)
        need = _ws_need.get(key)
        if need is None:
            need = _ws_need[key] = L.ggq_workspace_bytes(*key)
        ws = _backend.workspace(dev, need, stream)
        _lib.check(fn(key[0], data.data_ptr(), n_rows, k_dim, x_ptr, m, y.data_ptr(),
                      _backend.dtype_code(out_dtype), ws.data_ptr() if ws is not None else None,
                      ws.numel() if ws is not None else 0, stream))
    finally:
        if prev != dev:
            torch.cuda.set_device(prev)
    return y.reshape(*x.shape[:-1], n_rows)


def matmul_q4_k(x, w, *, force_fused: bool = False):
    """Q4_K fused multiply (stands for src/gguf_jax/cute/q4_k.py:282-329)."""
    _check(x, w, (QT.Q4_K,))
    return fused_matmul(x, w)


def matmul_q5_k(x, w):
    """Q5_K fused multiply (src/gguf_jax/cute/q5_k.py:150-179)."""
    _check(x, w, (QT.Q5_K,))
    return fused_matmul(x, w)


def matmul_q6_k(x, w):
    """Q6_K fused multiply (src/gguf_jax/cute/q6_k.py:115-144)."""
    _check(x, w, (QT.Q6_K,))
    return fused_matmul(x, w)


def matmul_iq4_xs(x, w):
    """IQ4_XS fused multiply (src/gguf_jax/cute/iq4_xs.py:146-175): the tiled kernel, whose
    16-entry code book is applied with byte permutes on register-resident tables."""
    _check(x, w, (QT.IQ4_XS,))
    return fused_matmul(x, w)


def matmul_lowbit(x, w):
    """Fused multiply for the eight low-bit types (src/gguf_jax/cute/lowbit.py:675-712): the
    tiled kernel with the format's grid in shared memory and exact integer codes on the tensor cores."""
    _check(x, w, LOWBIT_TYPES)
    return fused_matmul(x, w)


def gemm_q4_k(x, w):
    """Q4_K tensor-core multiply for larger batches (src/gguf_jax/cute/q4_k_gemm.py:369-391);
    see :func:`fused_matmul` for which kernel a batch gets."""
    _check(x, w, (QT.Q4_K,))
    return fused_matmul(x, w)


def dequantize_q4_k(data, dtype=torch.float32):
    """Q4_K bytes ``(..., row_bytes)`` -> ``dtype`` ``(..., n)`` (src/gguf_jax/cute/q4_k.py:93-101)."""
    from . import quants

    return quants.dequantize(data, QT.Q4_K, dtype)


def register() -> None:
    """Kept for drop-in compatibility with ``gguf_jax.cute.register``: the CUDA decode
    kernels are already the registered decoders, so there is nothing to replace."""
    return None
