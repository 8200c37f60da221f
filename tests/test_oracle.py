"""Pins the CPU oracle (oracle/ggq_oracle.c) against gguf.quants.dequantize -- the function
the reference's own tests treat as ground truth (tests/test_bitwise.py:65-101 there) -- and
against the committed fixtures.  CPU only."""
import gguf
import numpy as np
import pytest
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import synth
from oracle import oracle as O

ALL_TYPES = sorted(set(gguf.quants._type_traits.keys()) | {QT.F16, QT.F32}, key=lambda t: t.name)
GOLDEN = np.load(__file__.replace("test_oracle.py", "golden/decode_golden.npz"))


def logical_shapes(qtype):
    n = max(GGML_QUANT_SIZES[qtype][0], 256)
    return [(n,), (4, 4 * n), (2, 3, n)]


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_c_oracle_random_bytes_bitwise(qtype):
    with np.errstate(all="ignore"):
        for i, shape in enumerate(logical_shapes(qtype)):
            byte_shape = gguf.quants.quant_shape_to_byte_shape(shape, qtype)
            data = np.random.default_rng(100 * int(qtype) + i).integers(0, 256, size=byte_shape, dtype=np.uint8)
            O.assert_bitwise_equal(O.c_dequantize(data, qtype), O.ref_dequantize(data, qtype), qtype.name)


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_c_oracle_quantized_floats_bitwise(qtype):
    rng = np.random.default_rng(0)
    shape = (8, max(GGML_QUANT_SIZES[qtype][0], 256))
    values = rng.normal(size=shape).astype(np.float32)
    values *= 10.0 ** rng.integers(-8, 8, size=(shape[0], 1)).astype(np.float32)
    values[0, :] = 0.0
    try:
        data = gguf.quants.quantize(values, qtype)
    except NotImplementedError:
        pytest.skip(f"gguf-py cannot quantize {qtype.name}")
    if data.dtype != np.uint8:
        data = np.ascontiguousarray(data).view(np.uint8)
    O.assert_bitwise_equal(O.c_dequantize(data, qtype), O.ref_dequantize(data, qtype), qtype.name)


@pytest.mark.parametrize("qtype", synth.BLOCK_QTYPES, ids=lambda t: t.name)
def test_c_oracle_matches_golden(qtype):
    for tag in ("rnd", "fin"):
        data = GOLDEN[f"{qtype.name}.{tag}.bytes"]
        want = GOLDEN[f"{qtype.name}.{tag}.f32bits"].view(np.float32)
        O.assert_bitwise_equal(O.c_dequantize(data, qtype), want, f"{qtype.name}.{tag}")


@pytest.mark.parametrize("qtype", synth.BLOCK_QTYPES, ids=lambda t: t.name)
def test_c_matmul_matches_golden_and_numpy(qtype):
    w, x, y = (GOLDEN[f"{qtype.name}.mm.{k}"] for k in ("w", "x", "y"))
    got = O.c_matmul(O.bf16_bits(x), w, qtype)
    assert O.rel_l2(got, y) < 1e-6
    got32 = O.c_matmul(O.bf16_bits(x), w, qtype, plain_f32=True)
    assert O.rel_l2(got32, y) < 1e-5
    ref = O.ref_matmul(O.bf16_bits(x), w, qtype)
    assert O.rel_l2(ref, y) < 1e-5


def test_ksigns_formula_matches_gguf():
    ks = np.frombuffer(gguf.quants.IQ2_XXS.ksigns, dtype=np.uint8)
    i = np.arange(128, dtype=np.uint32)
    parity = np.array([bin(v).count("1") & 1 for v in range(128)], dtype=np.uint32)
    assert np.array_equal(ks, (i | (parity << 7)).astype(np.uint8))


def test_bf16_helpers_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], dtype=np.float32)
    bits = O.bf16_bits(x)
    import ml_dtypes
    want = x.astype(ml_dtypes.bfloat16).view(np.uint16)
    assert np.array_equal(bits, want)
    assert np.array_equal(O.bf16_to_f32(bits), want.view(ml_dtypes.bfloat16).astype(np.float32))


def test_synthetic_weights_decode_finite():
    for qt in synth.BLOCK_QTYPES:
        v = O.c_dequantize(synth.make_weight_bytes(4, 512, qt, seed=3), qt)
        assert np.isfinite(v).all(), qt.name
