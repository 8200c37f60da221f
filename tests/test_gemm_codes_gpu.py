"""The integer-code tcgen05 GEMM behind ggq_gemm for Q4_K / Q5_K / Q6_K (gemm_codes.cu): exact bf16 code
operands, one TMEM slot per scale group, float32 scales applied by the epilogue.  Against the CPU oracle
on a B200.  Nothing is rounded before the output, so the float32 result is within 2e-5 relative L2 of the
oracle's double-accumulated product (the tf32 kernel that serves the other formats is at 3e-4), a one-hot
activation returns the decoded weight exactly, and a launch is deterministic, K split included."""
import ctypes

import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import _lib, kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
CODE_TYPES = [QT.Q4_K, QT.Q5_K, QT.Q6_K]


@pytest.fixture(autouse=True)
def _tcgen05_kernel_for_every_batch(monkeypatch):
    # ggq_gemm would otherwise hand these formats to the batch-major mma.sync kernel (up to 32 rows) or to the
    # bf16-weight tcgen05 kernel (above)
    monkeypatch.setenv("GGQ_GEMM_KERNEL", "codes")


def run(x, wb, qtype, out_dtype=torch.float32):
    n, k = wb.shape[0], x.shape[1]
    w = gj.QuantizedArray.from_bytes(wb, qtype, shape=(n, k), device="cuda")
    return kernels.fused_matmul(torch.from_numpy(x).cuda().to(torch.bfloat16), w, out_dtype=out_dtype).float().cpu().numpy()


def status_word():
    word = ctypes.c_int32(0)
    rc = _lib.lib().ggq_read_status(torch.cuda.current_device(), ctypes.byref(word))
    return rc, word.value


@pytest.mark.parametrize("qtype", CODE_TYPES, ids=lambda t: t.name)
def test_matches_oracle_across_tile_edges(qtype):
    # K multiples of 2048 keep Q6_K rows 16-byte aligned; N and M ragged against the 128 x 64 tile
    for n, k in [(128, 2048), (200, 4096), (1100, 2048)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=n)
        for m in (17, 63, 64, 65, 130, 300):
            x = synth.make_x(m, k, seed=m)
            ref = O.c_matmul(O.bf16_bits(x), wb, qtype)
            got = run(x, wb, qtype)
            assert O.rel_l2(got, ref) <= 2e-5, (qtype.name, n, k, m, O.rel_l2(got, ref))
            got16 = run(x, wb, qtype, torch.bfloat16)
            np.testing.assert_allclose(got16, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
    assert status_word() == (0, 0)


@pytest.mark.parametrize("qtype", CODE_TYPES, ids=lambda t: t.name)
def test_one_hot_rows_return_the_weight_exactly(qtype):
    n, k = 130, 2048
    wb = synth.make_weight_bytes(n, k, qtype, seed=2)
    dense = O.ref_dequantize(wb, qtype)
    cols = list(range(0, 256, 5)) + [1000, 2047]
    x = np.zeros((len(cols), k), dtype=np.float32)
    x[np.arange(len(cols)), cols] = 1.0
    got = run(x, wb, qtype)
    assert np.array_equal(got, dense[:, cols].T)


def test_activation_rows_of_different_magnitude():
    n, k, m = 256, 2048, 20
    wb = synth.make_weight_bytes(n, k, QT.Q4_K, seed=5)
    x = synth.make_x(m, k, seed=5)
    x *= (2.0 ** np.linspace(-60, 60, m, dtype=np.float32)).reshape(m, 1)
    ref = O.c_matmul(O.bf16_bits(x), wb, QT.Q4_K)
    got = run(x, wb, QT.Q4_K)
    for r in range(m):
        assert O.rel_l2(got[r], ref[r]) <= 2e-5, r


def test_k_split_is_deterministic_and_leaves_the_scratch_clean():
    n, k, m = 512, 16 * 256, 48          # four row tiles: the launch cuts K into ranges
    wb = synth.make_weight_bytes(n, k, QT.Q6_K, seed=21)
    x = synth.make_x(m, k, seed=22)
    ref = O.c_matmul(O.bf16_bits(x), wb, QT.Q6_K)
    first = run(x, wb, QT.Q6_K)
    assert O.rel_l2(first, ref) <= 2e-5
    x1 = synth.make_x(1, k, seed=23)
    ref1 = O.c_matmul(O.bf16_bits(x1), wb, QT.Q6_K)
    for _ in range(3):
        assert O.rel_l2(run(x1, wb, QT.Q6_K), ref1) <= 2e-5       # the batch-1 kernel shares the counter area
        again = run(x, wb, QT.Q6_K)
        assert np.array_equal(again.view(np.uint32), first.view(np.uint32))
    assert status_word() == (0, 0)


def test_config_shapes_sampled_rows():
    """Llama-3-8B shapes of the Q5_K / Q6_K GEMM configuration at 32 and 128 tokens: 128 sampled rows."""
    for qtype, n, k in [(QT.Q5_K, 4096, 4096), (QT.Q6_K, 14336, 4096), (QT.Q6_K, 4096, 14336)]:
        wb = synth.make_weight_bytes(n, k, qtype, seed=9)
        w = gj.QuantizedArray.from_bytes(wb, qtype, shape=(n, k), device="cuda")
        rows = np.sort(np.random.default_rng(4).choice(n, size=128, replace=False))
        for m in (32, 128):
            x = synth.make_x(m, k, seed=m)
            ref = O.c_matmul(O.bf16_bits(x), wb[rows], qtype)
            got = kernels.fused_matmul(torch.from_numpy(x).cuda().to(torch.bfloat16), w, out_dtype=torch.float32).cpu().numpy()[:, rows]
            assert O.rel_l2(got, ref) <= 2e-5, (qtype.name, n, k, m)
