"""CPU oracle for the dequantize-and-multiply path.  TEST INFRASTRUCTURE ONLY.

Two independent checkers live here:

* ``ref_dequantize`` -- ``gguf.quants.dequantize`` from the third-party package gguf
  0.19.0, the exact oracle the reference's own tests compare against
  (tests/test_bitwise.py:65-101 in the reference).  The reference's decoders
  (src/gguf_jax/quants.py:125-712) mirror it operation for operation.
* the C restatement in ``ggq_oracle.c`` (``c_dequantize``, ``c_matmul``), pinned against
  the first by tests/test_oracle.py and the fixtures under tests/golden/.  It exists so
  that the large shapes (8192 x 28672) can be checked and timed without a dense float32
  temporary, and so that the CPU baseline is compiled code using every host core.

``ref_matmul`` restates ``_dequant_forward`` (src/gguf_jax/_matmul.py:195-201) with
``blocks == 1`` at dtype float32: ``x.astype(float32) @ dequantize(w).T``.

The product path (gguf_jax_b200) must never import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
from gguf import quants as _gq
from gguf.constants import GGML_QUANT_SIZES, GGMLQuantizationType as QT

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libggq_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ggq_oracle.c with the Makefile beside it (gcc + OpenMP)."""
    if force or not os.path.exists(_SO) or (
            os.path.getmtime(_SO) < os.path.getmtime(os.path.join(_HERE, "ggq_oracle.c"))):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def tables_blob() -> np.ndarray:
    """Codebook blob in the layout include/ggq.h documents, read from gguf.quants.

    Same sources as the reference: grids through ``init_grid`` and ``ksigns``-free sign
    handling (src/gguf_jax/quants.py:476-483); the 16-entry value tables from the
    ``kvalues`` class attributes.
    """
    parts = []
    for cls in (_gq.IQ2_XXS, _gq.IQ2_XS, _gq.IQ2_S, _gq.IQ3_XXS, _gq.IQ3_S):
        cls.init_grid()
        g = np.asarray(cls.grid).reshape(cls.grid_shape)
        assert g.min() >= 0 and g.max() <= 255 and np.all(g == np.round(g))
        parts.append(g.astype(np.uint8).reshape(-1))
    _gq.IQ1_S.init_grid()
    g = np.asarray(_gq.IQ1_S.grid).reshape(_gq.IQ1_S.grid_shape)
    parts.append(g.astype(np.int8).reshape(-1).view(np.uint8))
    parts.append(np.array(_gq.IQ4_NL.kvalues, dtype=np.int8).view(np.uint8))
    parts.append(np.array(_gq.MXFP4.kvalues, dtype=np.int8).view(np.uint8))
    return np.ascontiguousarray(np.concatenate(parts))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        L.ggq_oracle_set_tables.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        L.ggq_oracle_dequant.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        for name in ("ggq_oracle_matmul", "ggq_oracle_matmul_f32"):
            getattr(L, name).argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.ggq_oracle_type_info.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                           ctypes.POINTER(ctypes.c_int)]
        blob = tables_blob()
        assert blob.nbytes == L.ggq_oracle_tables_bytes()
        assert L.ggq_oracle_set_tables(blob.ctypes.data, blob.nbytes) == 0
        _lib = L
    return _lib


def threads() -> int:
    return int(lib().ggq_oracle_threads())


def set_threads(n: int) -> int:
    """Use ``n`` OpenMP threads from now on (launchers like torchrun export OMP_NUM_THREADS=1);
    returns the count in effect."""
    return int(lib().ggq_oracle_set_threads(int(n)))


# ---------------------------------------------------------------------------------------
# decode

def ref_dequantize(data: np.ndarray, qtype: QT) -> np.ndarray:
    """``gguf.quants.dequantize`` -> float32 (the reference's oracle)."""
    return _gq.dequantize(np.ascontiguousarray(data), qtype)


def c_dequantize(data: np.ndarray, qtype: QT) -> np.ndarray:
    """C restatement of dequantize (src/gguf_jax/quants.py:733-745): byte-shaped uint8
    ``(..., row_bytes)`` -> float32 ``(..., n)``."""
    data = np.ascontiguousarray(data)
    if qtype in (QT.F32, QT.F16, QT.BF16):
        bs, ts = 1, {QT.F32: 4, QT.F16: 2, QT.BF16: 2}[qtype]
    else:
        bs, ts = GGML_QUANT_SIZES[qtype]
    if data.dtype != np.uint8:
        data = data.view(np.uint8)
    if data.shape[-1] % ts:
        raise ValueError(f"row of {data.shape[-1]} bytes is not a multiple of {ts}")
    nb = data.size // ts
    out = np.empty(nb * bs, dtype=np.float32)
    rc = lib().ggq_oracle_dequant(int(qtype), data.ctypes.data, nb, out.ctypes.data)
    if rc:
        raise NotImplementedError(f"oracle cannot decode {qtype!r} (rc={rc})")
    return out.reshape(*data.shape[:-1], data.shape[-1] // ts * bs)


# ---------------------------------------------------------------------------------------
# matmul

def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even, NaN kept."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + r) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), out)
    return out


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def ref_matmul(x_bf16_bits: np.ndarray, w_bytes: np.ndarray, qtype: QT, dtype=np.float32) -> np.ndarray:
    """numpy restatement of _dequant_forward (src/gguf_jax/_matmul.py:195-201)."""
    W = ref_dequantize(w_bytes, qtype).astype(dtype)
    return bf16_to_f32(x_bf16_bits).astype(dtype) @ W.T


def c_matmul(x_bf16_bits: np.ndarray, w_bytes: np.ndarray, qtype: QT, *, plain_f32: bool = False) -> np.ndarray:
    """C restatement of the same product, fused per row; float32 out.

    ``plain_f32=False`` accumulates each dot product in double and rounds once;
    ``plain_f32=True`` accumulates in float32 (the timed CPU-baseline variant).
    """
    w_bytes = np.ascontiguousarray(w_bytes)
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    bs, ts = GGML_QUANT_SIZES[qtype]
    N = w_bytes.shape[0]
    K = w_bytes.shape[1] // ts * bs
    M = x.shape[0]
    assert x.shape == (M, K)
    y = np.empty((M, N), dtype=np.float32)
    fn = lib().ggq_oracle_matmul_f32 if plain_f32 else lib().ggq_oracle_matmul
    rc = fn(int(qtype), w_bytes.ctypes.data, N, K, x.ctypes.data, M, y.ctypes.data)
    if rc:
        raise RuntimeError(f"oracle matmul failed rc={rc}")
    return y


def rel_l2(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def assert_bitwise_equal(ours: np.ndarray, ref: np.ndarray, what: str = "") -> None:
    """Raw float32 bit patterns must match; only positions where BOTH are NaN are exempt
    (the reference's rule, tests/test_bitwise.py:27-49)."""
    assert ours.shape == ref.shape, (ours.shape, ref.shape)
    assert ours.dtype == np.float32 and ref.dtype == np.float32
    a = ours.view(np.uint32)
    b = ref.view(np.uint32)
    bad = (a != b) & ~(np.isnan(ours) & np.isnan(ref))
    if bad.any():
        idx = tuple(int(i[0]) for i in np.nonzero(bad))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} mismatched; first at {idx}: "
            f"ours={ours[idx]!r} (0x{a[idx]:08x}) ref={ref[idx]!r} (0x{b[idx]:08x})")
