"""ctypes binding of libggq_b200.so, the C-ABI library declared in include/ggq.h.

There is no CPU or eager fallback: if the library is missing or a call fails, the error
is raised to the caller.
"""
from __future__ import annotations

import ctypes
import os
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# GGQ_B200_LIB overrides the in-tree library (for trying out a differently built copy).
LIB_PATH = os.environ.get("GGQ_B200_LIB") or os.path.join(_HERE, "libggq_b200.so")

GGQ_F32, GGQ_BF16, GGQ_F16 = 0, 1, 2

_lib = None
_lock = threading.RLock()  # ensure_tables() calls lib() while holding it
_tables_done: set[int] = set()

# name -> (restype, argtypes); one entry per declaration in include/ggq.h
SIGNATURES = {
    "ggq_version": (ctypes.c_int32, []),
    "ggq_last_error": (ctypes.c_char_p, []),
    "ggq_type_info": (ctypes.c_int32, [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32),
                                       ctypes.POINTER(ctypes.c_int32)]),
    "ggq_tables_bytes": (ctypes.c_size_t, []),
    "ggq_set_tables": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t]),
    "ggq_init": (ctypes.c_int32, [ctypes.c_int32]),
    "ggq_dequant": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                     ctypes.c_int32, ctypes.c_void_p]),
    "ggq_has_fused": (ctypes.c_int32, [ctypes.c_int32]),
    "ggq_fused_batch_limit": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_int64, ctypes.c_int64]),
    "ggq_gemv_max_batch": (ctypes.c_int32, []),
    "ggq_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32]),
    "ggq_gemv": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                  ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32,
                                  ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "ggq_gemm": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                  ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32,
                                  ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "ggq_gemv_sharded": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_void_p, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p),
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32,
                                          ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                          ctypes.c_size_t, ctypes.c_void_p]),
    "ggq_gemm_sharded": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p),
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32,
                                          ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                          ctypes.c_size_t, ctypes.c_void_p]),
    "ggq_gemv_sharded_tagged": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                                 ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                                 ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_int32,
                                                 ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t,
                                                 ctypes.c_void_p]),
    "ggq_gemv_q4k_static": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]),
    "ggq_read_status": (ctypes.c_int32, [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)]),
    "ggq_stage_host": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
}


class GGQError(RuntimeError):
    """A non-zero status from the C ABI."""

    def __init__(self, status: int, message: str):
        super().__init__(f"ggq status {status}: {message}")
        self.status = status


def lib() -> ctypes.CDLL:
    """Load libggq_b200.so (built by ``python -m gguf_jax_b200.build``)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m gguf_jax_b200.build` "
                        "(nvcc, sm_100a). There is no CPU fallback.")
                L = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(L, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = L
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise GGQError(status, lib().ggq_last_error().decode("utf-8", "replace"))


def tables_blob() -> np.ndarray:
    """Codebook blob for ggq_set_tables, read from gguf.quants at run time.

    The reference takes the same tables from the same place
    (src/gguf_jax/quants.py:476-483, cute/lowbit.py:401-420); none is transcribed here.
    """
    from gguf import quants as gq

    parts = []
    for cls in (gq.IQ2_XXS, gq.IQ2_XS, gq.IQ2_S, gq.IQ3_XXS, gq.IQ3_S):
        cls.init_grid()
        parts.append(np.asarray(cls.grid).reshape(cls.grid_shape).astype(np.uint8).reshape(-1))
    gq.IQ1_S.init_grid()
    parts.append(np.asarray(gq.IQ1_S.grid).reshape(gq.IQ1_S.grid_shape).astype(np.int8).reshape(-1).view(np.uint8))
    parts.append(np.array(gq.IQ4_NL.kvalues, dtype=np.int8).view(np.uint8))
    parts.append(np.array(gq.MXFP4.kvalues, dtype=np.int8).view(np.uint8))
    blob = np.ascontiguousarray(np.concatenate(parts))
    return blob


def ensure_tables(device_index: int) -> None:
    """Upload the codebooks to ``device_index`` once per process."""
    if device_index in _tables_done:
        return
    with _lock:
        if device_index in _tables_done:
            return
        L = lib()
        blob = tables_blob()
        if blob.nbytes != L.ggq_tables_bytes():
            raise RuntimeError(f"codebook blob is {blob.nbytes} bytes, library expects {L.ggq_tables_bytes()}")
        check(L.ggq_set_tables(device_index, blob.ctypes.data, blob.nbytes))
        check(L.ggq_init(device_index))      # the status word that bounded device-side waits raise, outside any capture
        _tables_done.add(device_index)
