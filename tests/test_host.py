"""Host-side logic that needs no GPU: the QuantizedArray pytree, the registry, the router's
argument checks and block counting.  Mirrors the CPU parts of the reference's
tests/test_array.py and tests/test_matmul.py."""
import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT
from torch.utils import _pytree

import gguf
import gguf_jax_b200 as gj
from gguf_jax_b200 import _matmul as mm
from gguf_jax_b200 import quants, synth


def test_public_names_match_reference():
    assert set(gj.__all__) == {
        "GGMLQuantizationType", "GGUFFile", "QuantizedArray", "dequant_matmul", "dequantize",
        "dequantize_blocks", "fused_batch_limit", "fused_types", "load_gguf", "matmul", "quantize",
        "register_dequant", "supported_types"}
    from gguf_jax_b200 import cute
    assert set(cute.__all__) == {
        "LOWBIT_TYPES", "dequantize_q4_k", "gemm_q4_k", "matmul_iq4_xs", "matmul_lowbit", "matmul_q4_k",
        "matmul_q5_k", "matmul_q6_k", "register"}


def test_supported_types_match_gguf():
    ref = set(gguf.quants._type_traits.keys()) | {QT.F16, QT.F32}
    assert set(gj.supported_types()) == ref


def test_pytree_has_one_uint8_leaf():
    w = synth.make_weight(4, 512, QT.Q4_K, device="cpu")
    leaves, spec = _pytree.tree_flatten({"w": w, "b": torch.zeros(3)})
    q_leaves = [l for l in leaves if l.dtype == torch.uint8]
    assert len(leaves) == 2 and len(q_leaves) == 1 and q_leaves[0].shape == (4, 288)
    back = _pytree.tree_unflatten(leaves, spec)
    assert isinstance(back["w"], gj.QuantizedArray) and back["w"].shape == (4, 512) and back["w"].qtype == QT.Q4_K
    mapped = _pytree.tree_map(lambda t: t.clone(), w)
    assert isinstance(mapped, gj.QuantizedArray) and torch.equal(mapped.data, w.data)


def test_shape_inference_and_repr():
    data = np.zeros((2, 3, 34 * 4), dtype=np.uint8)
    a = gj.QuantizedArray.from_bytes(data, QT.Q8_0, device="cpu")
    assert a.shape == (2, 3, 128) and a.ndim == 3 and a.size == 768 and a.nbytes == data.nbytes
    assert "Q8_0" in repr(a) and "bfloat16" in repr(a)
    assert a.astype(torch.float32).dtype == torch.float32
    assert a.astype("float16").dtype == torch.float16


def test_native_integer_passthrough():
    a = gj.QuantizedArray.from_bytes(np.arange(6, dtype=np.int32).reshape(2, 3), QT.I32, device="cpu")
    assert a.dequantize().dtype == torch.int32 and a.dequantize().tolist() == [[0, 1, 2], [3, 4, 5]]


def test_non_uint8_payload_raises():
    with pytest.raises(ValueError):
        gj.QuantizedArray.from_bytes(np.zeros((2, 34), dtype=np.int8), QT.Q8_0, device="cpu")


def test_bad_byte_count_raises():
    with pytest.raises(ValueError):
        gj.dequantize(torch.zeros(3, dtype=torch.uint8), QT.Q8_0)
    with pytest.raises(ValueError):
        gj.dequantize_blocks(torch.zeros((2, 33), dtype=torch.uint8), QT.Q8_0)
    with pytest.raises(NotImplementedError):
        gj.dequantize_blocks(torch.zeros((2, 4), dtype=torch.uint8), QT.I32)


def test_register_dequant_contract():
    with pytest.raises(ValueError):
        gj.register_dequant(QT.Q4_K, lambda b, d: b)
    saved = quants._DEQUANT[QT.Q8_0]
    try:
        gj.register_dequant(QT.Q8_0, lambda b, d: torch.ones((b.shape[0], 32), dtype=d), override=True)
        out = gj.dequantize(torch.zeros((2, 34), dtype=torch.uint8, device="cpu"), QT.Q8_0, torch.float16)
        assert out.shape == (2, 32) and out.dtype == torch.float16 and bool((out == 1).all())
    finally:
        gj.register_dequant(QT.Q8_0, saved, override=True)


def test_no_cpu_fallback():
    w = synth.make_weight(4, 512, QT.Q4_K, device="cpu")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        w.dequantize()
    x = torch.zeros((1, 512), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        gj.matmul(x, w)


def test_matmul_argument_errors(built_lib):
    w = synth.make_weight(4, 512, QT.Q4_K, device="cpu")
    x = torch.zeros((1, 512), dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        gj.matmul(x, torch.zeros(4, 512))
    with pytest.raises(ValueError):
        gj.matmul(torch.zeros((1, 256), dtype=torch.bfloat16), w)
    w3 = gj.QuantizedArray.from_bytes(np.zeros((2, 2, 144), np.uint8), QT.Q4_K, device="cpu")
    with pytest.raises(ValueError):
        gj.matmul(torch.zeros((1, 256), dtype=torch.bfloat16), w3)


def test_router_caps(built_lib):
    fused = set(gj.fused_types())
    reference_fused = {QT.Q4_K, QT.Q5_K, QT.Q6_K, QT.IQ4_XS, QT.Q2_K, QT.IQ1_M, QT.IQ2_XXS, QT.IQ2_XS,
                       QT.IQ2_S, QT.IQ3_XXS, QT.IQ3_S, QT.IQ1_S}
    assert reference_fused <= fused
    for qt in fused:
        assert gj.fused_batch_limit(synth.make_weight(8, 512, qt, device="cpu")) >= 1, qt.name
    f16 = gj.QuantizedArray.from_bytes(np.zeros((4, 64), np.uint8), QT.F16, shape=(4, 32), device="cpu")
    assert gj.fused_batch_limit(f16) == 0


@pytest.mark.parametrize("rows,cols,budget", [(4096, 4096, 512 << 20), (128256, 8192, 512 << 20),
                                              (1000, 512, 1 << 16), (7, 512, 1024)])
def test_block_count_divides(rows, cols, budget):
    n = mm._block_count(rows, cols, budget)
    assert rows % n == 0
    assert n == rows or 4 * (rows // n) * cols <= budget
    if 4 * rows * cols <= budget:
        assert n == 1
