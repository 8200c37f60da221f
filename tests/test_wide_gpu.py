"""The batch-major fused multiply (gemv_wide.cu: Q4_K, Q5_K, Q6_K, 5..32 batch rows per launch, larger batches
in slices) against the CPU oracle on a B200, through the public wrappers / the C ABI.

Bars: float32 output within 2e-5 relative L2 of the oracle's double-accumulated product (nothing but float32
summation order separates them); bf16 output = that float32 result rounded once, within the reference's
elementwise rtol = 1e-2, atol = 1e-2 max|ref|; a one-hot activation (a power of two) returns the decoded
weight times the activation exactly at every position of a superblock; a launch is repeatable bit for bit."""
import ctypes

import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import _lib, kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

WIDE = [QT.Q4_K, QT.Q5_K, QT.Q6_K]


@pytest.fixture(autouse=True, params=["tma_boxes", "cp_async"])
def _batch_major_kernel_for_every_batch(monkeypatch, request):
    # above 32 rows ggq_gemm would otherwise pick the bf16-weight tcgen05 kernel; every test runs with the weight
    # slots copied as TMA boxes and as per-lane cp.async (the library reads the switch on every call)
    monkeypatch.setenv("GGQ_GEMM_KERNEL", "wide")
    monkeypatch.setenv("GGQ_WIDE_TMA", "1" if request.param == "tma_boxes" else "0")
    # likewise the output stores: 16-byte runs (default) with the boxes, element-wise with cp.async
    monkeypatch.setenv("GGQ_WIDE_VEC_STORE", "1" if request.param == "tma_boxes" else "0")


BIG = (6144, 6144)            # 21 to 31 MB in these formats: above the size from which ggq_gemv picks this kernel


def on_device(wb, qt, n, k):
    return gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device="cuda")


def to_x(x):
    return torch.from_numpy(x).cuda().to(torch.bfloat16)


def wide_direct(x, w, qt, n, k, out_dtype=torch.float32):
    """ggq_gemm with the workspace and the kernel pinned: the batch-major kernel in slices of 32 rows, whatever the
    weight's size (ggq_gemv would pick it only for large weights)."""
    L = _lib.lib()
    m = x.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device="cuda")
    ws = torch.zeros(L.ggq_workspace_bytes(int(qt), n, k, max(m, 17)), dtype=torch.uint8, device="cuda")
    code = {torch.float32: _lib.GGQ_F32, torch.bfloat16: _lib.GGQ_BF16}[out_dtype]
    _lib.check(L.ggq_gemm(int(qt), w.data.data_ptr(), n, k, x.data_ptr(), m, y.data_ptr(), code, ws.data_ptr(), ws.numel(),
                          torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(ws[128 * 1024:4 * 1024 * 1024].view(torch.int32).abs().max()) == 0      # arrival counters are left at zero
    return y


@pytest.mark.parametrize("qtype", WIDE, ids=lambda t: t.name)
def test_batches_and_ragged_shapes(qtype):
    # K multiples of 2048 keep rows 16-byte aligned for every format; N ragged against 16 and 256, one to
    # several row blocks, fewer steps than CTAs and more
    for n, k in [(200, 2048), (33, 4096), (1100, 6144), (2600, 2048)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=n)
        w = on_device(wb, qtype, n, k)
        for m in (1, 5, 8, 9, 16, 17, 31, 32, 33, 70):
            xb = synth.make_x(m, k, seed=m)
            ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
            got32 = wide_direct(to_x(xb), w, qtype, n, k).cpu().numpy()
            assert O.rel_l2(got32, ref) <= 2e-5, (qtype.name, n, k, m)
            got16 = wide_direct(to_x(xb), w, qtype, n, k, torch.bfloat16).float().cpu().numpy()
            np.testing.assert_allclose(got16, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
            assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("qtype", WIDE, ids=lambda t: t.name)
def test_one_hot_is_exact_at_every_position_of_a_superblock(qtype):
    n, k = 64, 4096
    wb = synth.make_weight_bytes(n, k, qtype, seed=7)
    w = on_device(wb, qtype, n, k)
    dense = O.ref_dequantize(wb, qtype)
    cols = list(range(256, 512)) + [0, 700, 1023, 1024, k - 1]       # an odd superblock (2 mod 4 for Q6_K) and strays
    for lo in range(0, len(cols), 29):
        sel = cols[lo:lo + 29]
        for val in (1.0, -4.0):
            x = np.zeros((len(sel), k), dtype=np.float32)
            x[np.arange(len(sel)), sel] = val
            got = wide_direct(to_x(x), w, qtype, n, k).cpu().numpy()
            want = dense[:, sel].T.astype(np.float32) * np.float32(val)
            assert np.array_equal(got, want), (qtype.name, lo, val)


@pytest.mark.parametrize("qtype", WIDE, ids=lambda t: t.name)
def test_batch_rows_of_different_magnitude(qtype):
    # every batch row has its own power-of-two scale; rows far outside the usual range take another exponent
    n, k, m = 96, 2048, 12
    wb = synth.make_weight_bytes(n, k, qtype, seed=3)
    w = on_device(wb, qtype, n, k)
    xb = synth.make_x(m, k, seed=3)
    for i, e in enumerate([-70, -40, -20, -3, 0, 0, 7, 25, 35, 70, 100, 0]):
        xb[i] *= np.float32(2.0) ** e
    xb[11] = 0.0
    xb = torch.from_numpy(xb).to(torch.bfloat16).float().numpy()
    ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
    got = wide_direct(to_x(xb), w, qtype, n, k).cpu().numpy()
    for i in range(m):
        assert O.rel_l2(got[i:i + 1], ref[i:i + 1]) <= 2e-5 or not np.any(ref[i]), (qtype.name, i)
    assert not np.any(got[11])


def test_shortest_rows():
    # one and two superblocks per row (Q6_K rows are 16-byte aligned only from eight superblocks on)
    for qtype, n, k in [(QT.Q4_K, 64, 256), (QT.Q4_K, 700, 512), (QT.Q5_K, 300, 512), (QT.Q5_K, 40, 256), (QT.Q6_K, 130, 2048)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=k)
        w = on_device(wb, qtype, n, k)
        for m in (3, 20):
            xb = synth.make_x(m, k, seed=m)
            ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
            assert O.rel_l2(wide_direct(to_x(xb), w, qtype, n, k).cpu().numpy(), ref) <= 2e-5, (qtype.name, n, k, m)


def test_repeatable_and_independent_of_other_batch_rows():
    qt, (n, k) = QT.Q4_K, (1100, 6144)
    wb = synth.make_weight_bytes(n, k, qt, seed=11)
    w = on_device(wb, qt, n, k)
    x = to_x(synth.make_x(32, k, seed=2))
    a = wide_direct(x, w, qt, n, k).cpu().numpy()
    b = wide_direct(x, w, qt, n, k).cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # a batch row's result does not depend on which other rows travel with it (same column tile count)
    c = wide_direct(x[8:32].contiguous(), w, qt, n, k).cpu().numpy()
    assert np.array_equal(a[8:32].view(np.uint32), c.view(np.uint32))


@pytest.mark.parametrize("qtype", WIDE, ids=lambda t: t.name)
def test_picked_by_the_small_batch_entry_for_large_weights(qtype):
    n, k = BIG
    wb = synth.make_weight_bytes(n, k, qtype, seed=5)
    w = on_device(wb, qtype, n, k)
    assert gj.fused_batch_limit(w) >= 32
    for m in (5, 16):
        xb = synth.make_x(m, k, seed=m)
        ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
        got = kernels.fused_matmul(to_x(xb), w, out_dtype=torch.float32).cpu().numpy()
        assert O.rel_l2(got, ref) <= 2e-5
        via_gemm = wide_direct(to_x(xb), w, qtype, n, k).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), via_gemm.view(np.uint32))        # the same kernel either way


@pytest.mark.parametrize("qtype", WIDE, ids=lambda t: t.name)
def test_benchmark_shape_sampled_rows(qtype):
    n, k = 8192, 28672
    w = synth.make_weight_on_device(n, k, qtype, seed=1, device="cuda")
    pick = np.sort(np.random.default_rng(0).choice(n, size=96, replace=False))
    idx = torch.from_numpy(pick).cuda()
    rows = w.data[idx].cpu().numpy()
    for m in (8, 16, 32):
        x = to_x(synth.make_x(m, k, seed=m))
        assert m <= gj.fused_batch_limit(w)            # large K-quant weights take the fused route up to 32 rows
        got = kernels.fused_matmul(x, w, out_dtype=torch.float32)
        ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), rows, qtype)
        assert O.rel_l2(got[:, idx].cpu().numpy(), ref) <= 2e-5, (qtype.name, m)
