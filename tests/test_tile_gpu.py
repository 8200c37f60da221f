"""The tiled fused multiply (gemv_tile.cu: Q4_K, Q2_K, IQ4_XS and the IQ1/IQ2/IQ3 grid formats, batch 1..16)
against the CPU oracle on a B200, through the public wrappers / the C ABI.

Bars: float32 output within 2e-5 relative L2 of the oracle's double-accumulated product (i.e. nothing
but float32 summation order separates them); bf16 output within 2e-3 relative L2 and the reference's
elementwise rtol = 1e-2, atol = 1e-2 max|ref|; a one-hot activation returns the decoded weight times
the activation exactly (for activations that are powers of two), at every position of a superblock; a launch
is deterministic."""
import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TILE = [QT.Q4_K, QT.Q5_K, QT.Q6_K, QT.Q2_K, QT.IQ4_XS, QT.IQ2_XXS, QT.IQ2_XS, QT.IQ2_S, QT.IQ3_XXS, QT.IQ3_S, QT.IQ1_S, QT.IQ1_M]
LOWBIT_SWEEP = [QT.Q2_K, QT.IQ1_S, QT.IQ1_M, QT.IQ2_XXS, QT.IQ2_XS, QT.IQ2_S, QT.IQ3_XXS, QT.IQ3_S, QT.IQ4_XS]


def on_device(wb, qt, n, k):
    return gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device="cuda")


def to_x(x):
    return torch.from_numpy(x).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("qtype", TILE, ids=lambda t: t.name)
def test_batches_and_ragged_shapes(qtype):
    # K multiples of 2048 keep rows 16-byte aligned for every format; N ragged against 16 and 32
    for n, k in [(200, 2048), (33, 4096), (1100, 6144)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=n)
        w = on_device(wb, qtype, n, k)
        for m in (1, 2, 3, 4, 5, 8, 9, 16):
            xb = synth.make_x(m, k, seed=m)
            ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
            got32 = kernels.fused_matmul(to_x(xb), w, out_dtype=torch.float32).cpu().numpy()
            assert O.rel_l2(got32, ref) <= 2e-5, (qtype.name, n, k, m)
            got16 = kernels.fused_matmul(to_x(xb), w).float().cpu().numpy()
            np.testing.assert_allclose(got16, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
            assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("qtype", TILE, ids=lambda t: t.name)
def test_one_hot_is_exact_at_every_position_of_a_superblock(qtype):
    n, k = 64, 2048
    wb = synth.make_weight_bytes(n, k, qtype, seed=7)
    w = on_device(wb, qtype, n, k)
    dense = O.ref_dequantize(wb, qtype)
    cols = list(range(256)) + [700, 1023, 1024, k - 1]
    for lo in range(0, len(cols), 8):
        sel = cols[lo:lo + 8]
        x = np.zeros((len(sel), k), dtype=np.float32)
        x[np.arange(len(sel)), sel] = 1.0
        got = kernels.fused_matmul(to_x(x), w, out_dtype=torch.float32).cpu().numpy()
        want = dense[:, sel].T.astype(np.float32)
        assert np.array_equal(got, want), (qtype.name, sel)
    x = np.zeros((1, k), dtype=np.float32)
    x[0, 77] = -4.0
    got = kernels.fused_matmul(to_x(x), w, out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(got[0], dense[:, 77] * np.float32(-4.0))


@pytest.mark.parametrize("qtype", [QT.Q4_K, QT.IQ3_S, QT.IQ1_M], ids=lambda t: t.name)
def test_activation_magnitudes(qtype):
    n, k = 96, 4096
    wb = synth.make_weight_bytes(n, k, qtype, seed=3)
    w = on_device(wb, qtype, n, k)
    base = synth.make_x(2, k, seed=3)
    for e in (-60, -20, 0, 20, 60):
        xb = base * np.float32(2.0 ** e)
        xb[1] *= np.float32(2.0 ** -7)          # the two batch rows differ in magnitude
        ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
        got = kernels.fused_matmul(to_x(xb), w, out_dtype=torch.float32).cpu().numpy()
        for r in range(2):
            assert O.rel_l2(got[r], ref[r]) <= 2e-5, (qtype.name, e, r)


@pytest.mark.parametrize("qtype", [QT.Q4_K, QT.IQ2_S], ids=lambda t: t.name)
def test_deterministic_and_row_slices_agree_with_the_whole(qtype):
    """The same launch twice gives the same bits (fixed summation order, no float atomics).  A launch on a
    row slice may cut K differently (the split adapts to the row count), so its rows agree with the
    whole-weight launch only up to float32 summation order: within 4e-6 relative to the row's scale."""
    n, k = 4096, 8192
    wb = synth.make_weight_bytes(n, k, qtype, seed=11)
    xb = synth.make_x(3, k, seed=12)
    whole = kernels.fused_matmul(to_x(xb), on_device(wb, qtype, n, k), out_dtype=torch.float32).cpu().numpy()
    again = kernels.fused_matmul(to_x(xb), on_device(wb, qtype, n, k), out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(again.view(np.uint32), whole.view(np.uint32))
    scale = np.abs(whole).max()
    for parts in (2, 8):
        rows = n // parts
        for p in (0, parts - 1):
            part = kernels.fused_matmul(to_x(xb), on_device(wb[p * rows:(p + 1) * rows], qtype, rows, k),
                                        out_dtype=torch.float32).cpu().numpy()
            np.testing.assert_allclose(part, whole[:, p * rows:(p + 1) * rows], rtol=0, atol=4e-6 * scale)


@pytest.mark.parametrize("qtype", LOWBIT_SWEEP, ids=lambda t: t.name)
def test_low_bit_sweep_shape_sampled_rows(qtype):
    """The 8192 x 28672 weight of the low-bit sweep at batch 1, 4 and 8: 256 sampled rows against the oracle.
    The relative-L2 bar on the bf16 result is applied from 512 outputs on: the output rounding alone
    contributes about 1.6e-3, so the statistic needs that many samples to sit below 2e-3 reliably."""
    n, k = 8192, 28672
    wb = synth.make_weight_bytes(n, k, qtype, seed=0)
    w = on_device(wb, qtype, n, k)
    rows = np.sort(np.random.default_rng(1).choice(n, size=256, replace=False))
    for m in (1, 4, 8):
        xb = synth.make_x(m, k, seed=m)
        ref = O.c_matmul(O.bf16_bits(xb), wb[rows], qtype)
        got32 = kernels.fused_matmul(to_x(xb), w, out_dtype=torch.float32).cpu().numpy()[:, rows]
        assert O.rel_l2(got32, ref) <= 2e-5, (qtype.name, m)
        got16 = gj.matmul(to_x(xb), w).float().cpu().numpy()[:, rows]
        if got16.size >= 512:
            assert O.rel_l2(got16, ref) <= 2e-3, (qtype.name, m)
        np.testing.assert_allclose(got16, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
