"""The bf16-weight tcgen05 GEMM behind ggq_gemm for Q4_K / Q5_K / Q6_K above 32 batch rows (gemm_bf16w.cu): weights
decoded to float32 exactly, rounded once to bf16, multiplied with the bf16 activations on the tensor cores with
float32 accumulation in tensor memory.  On a B200, through the C ABI.

Bars: against the same product computed in float64 from the bf16-rounded reference weights the float32 output is within
1e-4 relative L2 (the summation order differs, and for Q4_K / Q5_K the kernel's one-FMA decode is off by 2^-20 of a
weight before the bf16 rounding, which moves about one weight in a thousand to the neighbouring bf16 value; Q6_K is
exact: 1e-5); against the unrounded oracle the bf16 output is within the
reference's elementwise rtol = 1e-2, atol = 1e-2 max|ref| and 4e-3 relative L2; a launch is repeatable bit for bit, K
split included; the status word stays clean."""
import ctypes

import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import _lib, kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TYPES = [QT.Q4_K, QT.Q5_K, QT.Q6_K]


@pytest.fixture(autouse=True)
def _pin_the_kernel(monkeypatch):
    monkeypatch.setenv("GGQ_GEMM_KERNEL", "bf16w")       # also below 33 rows, where ggq_gemm would pick the batch-major kernel


def run(x, wb, qtype, out_dtype=torch.float32):
    n, k = wb.shape[0], x.shape[1]
    w = gj.QuantizedArray.from_bytes(wb, qtype, shape=(n, k), device="cuda")
    return kernels.fused_matmul(x, w, out_dtype=out_dtype)


def bf16_weight_product(x, wb, qtype):
    dense = torch.from_numpy(O.ref_dequantize(wb, qtype)).to(torch.bfloat16).double()
    return (x.cpu().double() @ dense.T).numpy()


def to_x(x):
    return torch.from_numpy(x).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("qtype", TYPES, ids=lambda t: t.name)
def test_equals_the_product_with_bf16_rounded_weights(qtype):
    # K multiples of 2048 keep Q6_K rows 16-byte aligned; N ragged against the 128-row tile, M against every batch tile
    for n, k in [(128, 2048), (200, 4096), (1100, 2048), (33, 6144)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=n)
        for m in (17, 32, 33, 64, 100, 128, 200, 256, 300, 600):         # up to 16 rows fused_matmul calls ggq_gemv
            x = to_x(synth.make_x(m, k, seed=m))
            got = run(x, wb, qtype).cpu().numpy()
            assert O.rel_l2(got, bf16_weight_product(x, wb, qtype)) <= (1e-5 if qtype == QT.Q6_K else 1e-4), (qtype.name, n, k, m)


@pytest.mark.parametrize("qtype", TYPES, ids=lambda t: t.name)
def test_against_the_unrounded_oracle(qtype):
    n, k, m = 1100, 4096, 96
    wb = synth.make_weight_bytes(n, k, qtype, seed=1)
    xb = synth.make_x(m, k, seed=2)
    ref = O.c_matmul(O.bf16_bits(xb), wb, qtype)
    got = run(to_x(xb), wb, qtype, torch.bfloat16).float().cpu().numpy()
    assert O.rel_l2(got, ref) <= 4e-3
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())


def test_k_split_is_repeatable_and_leaves_the_scratch_clean():
    qtype, n, k, m = QT.Q4_K, 256, 8192, 64            # two row tiles: K is split over many CTAs
    wb = synth.make_weight_bytes(n, k, qtype, seed=3)
    w = gj.QuantizedArray.from_bytes(wb, qtype, shape=(n, k), device="cuda")
    x = to_x(synth.make_x(m, k, seed=4))
    L = _lib.lib()
    ws = torch.zeros(L.ggq_workspace_bytes(int(qtype), n, k, m), dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(3):
        y = torch.empty((m, n), dtype=torch.float32, device="cuda")
        _lib.check(L.ggq_gemm(int(qtype), w.data.data_ptr(), n, k, x.data_ptr(), m, y.data_ptr(), _lib.GGQ_F32, ws.data_ptr(),
                              ws.numel(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        outs.append(y.cpu().numpy())
        assert int(ws[128 * 1024:4 * 1024 * 1024].view(torch.int32).abs().max()) == 0      # arrival counters back at zero
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert np.array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32))
    assert O.rel_l2(outs[0], bf16_weight_product(x, wb, qtype)) <= 1e-4
    word = ctypes.c_int32(-1)
    assert L.ggq_read_status(torch.cuda.current_device(), ctypes.byref(word)) == 0 and word.value == 0


@pytest.mark.parametrize("qtype", TYPES, ids=lambda t: t.name)
def test_router_takes_it_up_to_its_cap_on_large_weights(qtype, monkeypatch):
    monkeypatch.delenv("GGQ_GEMM_KERNEL")
    n, k = 6144, 6144
    w = synth.make_weight_on_device(n, k, qtype, seed=5, device="cuda")
    cap = gj.fused_batch_limit(w)
    assert cap == 256            # 48 row tiles: large, but not enough tiles for the 512-row cap
    pick = np.sort(np.random.default_rng(0).choice(n, size=64, replace=False))
    idx = torch.from_numpy(pick).cuda()
    rows = w.data[idx].cpu().numpy()
    for m in (33, cap):
        x = to_x(synth.make_x(m, k, seed=m))
        got = gj.matmul(x, w).float()[:, idx].cpu().numpy()
        ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), rows, qtype)
        assert O.rel_l2(got, ref) <= 4e-3
        np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
