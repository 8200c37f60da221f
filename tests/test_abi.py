"""The C-ABI library loads and exports every symbol include/ggq.h declares; the calls that
need no GPU behave as documented.  CPU only (nvcc cross-compiles without a device)."""
import ctypes
import os
import re

import pytest
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import _lib, quants

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ggq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ggq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built_lib):
    names = declared_symbols()
    assert len(names) >= 12
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), f"{name} declared in include/ggq.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table out of sync with the header"


def test_type_info_matches_gguf(built_lib):
    for qt in quants.supported_types():
        be, bb = ctypes.c_int32(), ctypes.c_int32()
        assert built_lib.ggq_type_info(int(qt), ctypes.byref(be), ctypes.byref(bb)) == 0
        assert (be.value, bb.value) == tuple(GGML_QUANT_SIZES[qt]), qt.name
    assert built_lib.ggq_type_info(int(QT.I32), None, None) != 0
    assert b"not decodable" in built_lib.ggq_last_error()


def test_tables_blob_size(built_lib):
    assert _lib.tables_blob().nbytes == built_lib.ggq_tables_bytes()


def test_caps_and_argument_errors_without_gpu(built_lib):
    assert built_lib.ggq_version() >= 100
    assert built_lib.ggq_gemv_max_batch() >= 1
    assert built_lib.ggq_has_fused(int(QT.Q4_K)) == 1
    assert built_lib.ggq_has_fused(int(QT.F16)) == 0
    assert built_lib.ggq_fused_batch_limit(int(QT.Q4_K), 4096, 4096) >= 1
    assert built_lib.ggq_fused_batch_limit(int(QT.F16), 4096, 4096) == 0
    assert built_lib.ggq_fused_batch_limit(int(QT.Q4_K), 4096, 100) == 0   # K not a block multiple
    # argument validation happens before any CUDA call
    assert built_lib.ggq_gemv(int(QT.Q4_K), None, 8, 100, None, 1, None, 1, None, 0, None) == 2  # BAD_SHAPE
    assert built_lib.ggq_gemv(int(QT.Q4_K), None, 8, 256, None, 99, None, 1, None, 0, None) == 2
    assert built_lib.ggq_gemv(int(QT.I8), None, 8, 256, None, 1, None, 1, None, 0, None) == 1    # BAD_QTYPE
    assert built_lib.ggq_dequant(int(QT.I8), None, 1, None, 0, None) == 1
    assert built_lib.ggq_dequant(int(QT.Q4_K), None, -1, None, 0, None) == 2
    with pytest.raises(_lib.GGQError):
        _lib.check(built_lib.ggq_dequant(int(QT.I8), None, 1, None, 0, None))


def test_sharded_entry_points_validate_before_any_cuda_call(built_lib):
    import ctypes
    ptrs = (ctypes.c_void_p * 8)()
    # rank outside the world, too many ranks
    assert built_lib.ggq_gemv_sharded(int(QT.Q4_K), None, 64, 256, None, 1, ptrs, ptrs, 9, 0, 576, 1, 0, None, 0, None) == 2
    assert built_lib.ggq_gemv_sharded(int(QT.Q4_K), None, 64, 256, None, 1, ptrs, ptrs, 2, 2, 128, 1, 0, None, 0, None) == 2
    # the shards do not fit the output
    assert built_lib.ggq_gemv_sharded(int(QT.Q4_K), None, 64, 256, None, 1, ptrs, ptrs, 2, 0, 100, 1, 0, None, 0, None) == 2
    assert built_lib.ggq_gemv_sharded_tagged(int(QT.Q4_K), None, 64, 256, None, None, 1, None, 0, 0, ptrs, None, 9, 0,
                                             576, None, 0, None) == 2
    assert built_lib.ggq_gemv_sharded_tagged(int(QT.I8), None, 64, 256, None, None, 1, None, 0, 0, ptrs, None, 2, 0,
                                             128, None, 0, None) == 1
    # neither plain nor tagged activations
    assert built_lib.ggq_gemv_sharded_tagged(int(QT.Q4_K), None, 64, 256, None, None, 1, None, 0, 0, ptrs, None, 2, 0,
                                             128, None, 0, None) == 3   # MISALIGNED (null pointer)
    assert b"null pointer" in built_lib.ggq_last_error()


def test_workspace_sizes(built_lib):
    # batch-1 tuned kernels: fixed partial area + one counter per 32 rows
    small = built_lib.ggq_workspace_bytes(int(QT.Q4_K), 4096, 4096, 1)
    assert small >= 131072 + 4096 // 32 * 4 and small % 256 == 0
    assert built_lib.ggq_workspace_bytes(int(QT.Q6_K), 4096, 4096, 1) == small
    assert built_lib.ggq_workspace_bytes(int(QT.Q5_K), 4096, 4096, 1) == small
    assert built_lib.ggq_workspace_bytes(int(QT.Q8_0), 4096, 4096, 1) == 0
    # the tensor-core kernel cuts K when there are few row tiles and then needs partial tiles
    # (sized without a device here, i.e. for 148 SMs)
    big = built_lib.ggq_workspace_bytes(int(QT.Q8_0), 1024, 8192, 64)
    assert big == 0 or big >= (4 << 20) + 2 * 64 * 1024 * 4
    # many row tiles: one K range per tile, no scratch
    assert built_lib.ggq_workspace_bytes(int(QT.Q8_0), 148 * 128 * 4, 1024, 64) == 0
