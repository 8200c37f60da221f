"""Decode kernel parity, through the C ABI on a B200: the float32 output must be bit-identical
to gguf.quants.dequantize for every decodable qtype (the reference's contract,
tests/test_bitwise.py there); bf16/f16 outputs are that result rounded once."""
import gguf
import ml_dtypes
import numpy as np
import pytest
import torch
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

ALL_TYPES = gj.supported_types()
GOLDEN = np.load(__file__.replace("test_decode_gpu.py", "golden/decode_golden.npz"))


def gpu_decode(data: np.ndarray, qtype, dtype=torch.float32) -> np.ndarray:
    out = gj.dequantize(torch.from_numpy(data).cuda(), qtype, dtype)
    if dtype == torch.float32:
        return out.cpu().numpy()
    return out.view(torch.int16).cpu().numpy().view(np.uint16)


def logical_shapes(qtype):
    n = max(GGML_QUANT_SIZES[qtype][0], 256)
    return [(n,), (4, 4 * n), (2, 3, n)]


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_random_bytes_bitwise(qtype):
    with np.errstate(all="ignore"):
        for i, shape in enumerate(logical_shapes(qtype)):
            byte_shape = gguf.quants.quant_shape_to_byte_shape(shape, qtype)
            data = np.random.default_rng(7 * int(qtype) + i).integers(0, 256, size=byte_shape, dtype=np.uint8)
            ours = gpu_decode(data, qtype)
            assert ours.shape == shape
            O.assert_bitwise_equal(ours, O.ref_dequantize(data, qtype), qtype.name)


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_many_blocks_bitwise_vs_c_oracle(qtype):
    """A size that spans many CTAs, checked against the C restatement."""
    bs, ts = GGML_QUANT_SIZES[qtype]
    nb = 40_001 if bs == 256 else 250_003
    data = np.random.default_rng(int(qtype)).integers(0, 256, size=(nb * ts,), dtype=np.uint8)
    O.assert_bitwise_equal(gpu_decode(data, qtype), O.c_dequantize(data, qtype), qtype.name)


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_quantized_floats_bitwise(qtype):
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
    with np.errstate(all="ignore"):
        O.assert_bitwise_equal(gpu_decode(data, qtype), O.ref_dequantize(data, qtype), qtype.name)


@pytest.mark.parametrize("qtype", synth.BLOCK_QTYPES, ids=lambda t: t.name)
def test_golden_fixtures(qtype):
    for tag in ("rnd", "fin"):
        data = GOLDEN[f"{qtype.name}.{tag}.bytes"]
        want = GOLDEN[f"{qtype.name}.{tag}.f32bits"].view(np.float32)
        O.assert_bitwise_equal(gpu_decode(data, qtype), want, f"{qtype.name}.{tag}")


@pytest.mark.parametrize("qtype", ALL_TYPES, ids=lambda t: t.name)
def test_narrow_outputs_are_the_f32_decode_rounded_once(qtype):
    bs, ts = GGML_QUANT_SIZES[qtype]
    data = synth.random_blocks(qtype, 64 * max(1, 256 // bs), seed=5) if qtype in synth.BLOCK_QTYPES else \
        np.random.default_rng(5).normal(size=(512,)).astype({QT.F32: np.float32, QT.F16: np.float16}.get(qtype, np.float32))
    if qtype == QT.BF16:
        data = O.bf16_bits(data)
    data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    f32 = O.ref_dequantize(data.view({QT.F32: np.float32, QT.F16: np.float16}.get(qtype, np.uint8))
                           if qtype in (QT.F32, QT.F16) else data, qtype).astype(np.float32).reshape(-1)
    finite = np.isfinite(f32)
    bf = gpu_decode(data, qtype, torch.bfloat16).reshape(-1)
    assert np.array_equal(bf[finite], f32.astype(ml_dtypes.bfloat16).view(np.uint16)[finite])
    with np.errstate(over="ignore"):
        want16 = f32.astype(np.float16).view(np.uint16)
    h = gpu_decode(data, qtype, torch.float16).reshape(-1)
    assert np.array_equal(h[finite], want16[finite])


def test_quantized_array_dequantize_and_cast():
    vals = np.random.default_rng(1).normal(size=(16, 256)).astype(np.float32)
    q = gj.quantize(vals, QT.Q8_0)
    assert q.data.is_cuda and q.shape == (16, 256)
    f32 = q.dequantize(torch.float32).cpu().numpy()
    O.assert_bitwise_equal(f32, O.ref_dequantize(q.data.cpu().numpy(), QT.Q8_0), "Q8_0")
    bf = q.dequantize()
    assert bf.dtype == torch.bfloat16
    assert torch.equal(bf, torch.from_numpy(f32).cuda().to(torch.bfloat16))
    assert np.abs(f32 - vals).max() < 0.05


def test_empty_input():
    out = gj.dequantize(torch.zeros((0, 144), dtype=torch.uint8, device="cuda"), QT.Q4_K)
    assert out.shape == (0, 256)
