"""Fused multiply parity on a B200, through the C ABI.

Pass criteria (stated in the tests): relative L2 error <= 2e-3 against the float32
dequant_matmul oracle; the reference's elementwise rtol=1e-2, atol=1e-2*max|ref|
(tests/test_cute.py there); and bitwise one-hot exactness -- x = e_k must return
bf16(float32 oracle weight[:, k]) (tests/test_cute.py:130-148, 412-424 there)."""
import numpy as np
import pytest
import torch
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import _matmul as mm
from gguf_jax_b200 import kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

REL_L2 = 2e-3
FUSED = gj.fused_types()
REFERENCE_FUSED = [QT.Q4_K, QT.Q5_K, QT.Q6_K, QT.IQ4_XS, QT.Q2_K, QT.IQ1_M, QT.IQ2_XXS, QT.IQ2_XS, QT.IQ2_S,
                   QT.IQ3_XXS, QT.IQ3_S, QT.IQ1_S]
GOLDEN = np.load(__file__.replace("test_matmul_gpu.py", "golden/decode_golden.npz"))


def to_x(x_f32: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(x_f32).cuda().to(torch.bfloat16)


def run_fused(x_f32, w_bytes, qtype, out_dtype=torch.bfloat16):
    n = w_bytes.shape[0]
    k = x_f32.shape[-1]
    w = gj.QuantizedArray.from_bytes(w_bytes, qtype, shape=(n, k))
    return kernels.fused_matmul(to_x(x_f32), w, out_dtype=out_dtype).float().cpu().numpy()


def check_close(got, ref):
    """bf16 result against the float32 oracle.  The L2 statistic is dominated by the output's
    own bf16 rounding (about 1.6e-3), so it is only meaningful over a few hundred outputs."""
    if ref.size >= 512:
        assert O.rel_l2(got, ref) <= REL_L2, O.rel_l2(got, ref)
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())


@pytest.mark.parametrize("qtype", FUSED, ids=lambda t: t.name)
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 12, 16])
def test_fused_matches_oracle(qtype, m):
    bs = GGML_QUANT_SIZES[qtype][0]
    n, k = 200, 11 * 256           # N not a tile multiple, rows only 2-byte aligned for most types
    w = synth.make_weight_bytes(n, k, qtype, seed=m)
    x = synth.make_x(m, k, seed=m)
    ref = O.c_matmul(O.bf16_bits(x), w, qtype)
    check_close(run_fused(x, w, qtype), ref)
    got32 = run_fused(x, w, qtype, torch.float32)
    assert O.rel_l2(got32, ref) <= 2e-5   # before the output rounding the kernel is float32-exact


@pytest.mark.parametrize("qtype", FUSED, ids=lambda t: t.name)
def test_golden_matmul(qtype):
    w, x, y = (GOLDEN[f"{qtype.name}.mm.{k}"] for k in ("w", "x", "y"))
    got32 = run_fused(x, w, qtype, torch.float32)
    assert O.rel_l2(got32, y) <= 2e-5
    # 24 outputs are too few for a stable L2 statistic on the bf16 result: check instead that
    # the bf16 result is the float32 result rounded once, plus the elementwise tolerance.
    got16 = run_fused(x, w, qtype)
    assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())
    np.testing.assert_allclose(got16, y, rtol=1e-2, atol=1e-2 * np.abs(y).max())


@pytest.mark.parametrize("qtype", FUSED, ids=lambda t: t.name)
def test_one_hot_exactness(qtype):
    bs = GGML_QUANT_SIZES[qtype][0]
    n, k = 24, 11 * 256
    w = synth.make_weight_bytes(n, k, qtype, seed=42)
    W = O.ref_dequantize(w, qtype)
    want = torch.from_numpy(W).to(torch.bfloat16).float().numpy()
    cols = [0, 1, 3, 4, 15, 16, 31, 32, 33, 63, 64, 127, 128, 255, 256, 257, 1000, k - 1]
    for lo in range(0, len(cols), 16):
        sel = cols[lo:lo + 16]
        x = np.zeros((len(sel), k), dtype=np.float32)
        x[np.arange(len(sel)), sel] = 1.0
        got = run_fused(x, w, qtype)
        assert np.array_equal(got, want[:, sel].T), qtype.name
    # and one at a time through the batch-1 path
    for c in (0, 33, k - 1):
        x = np.zeros((1, k), dtype=np.float32)
        x[0, c] = 1.0
        got = run_fused(x, w, qtype)
        assert np.array_equal(got[0], want[:, c]), (qtype.name, c)


@pytest.mark.parametrize("qtype", [QT.Q4_K, QT.Q6_K, QT.IQ2_XS], ids=lambda t: t.name)
def test_more_rows_than_resident_warps_and_short_rows(qtype):
    for n, k in ((20_000, 256), (3, 256), (1, 512), (4100, 1024)):
        w = synth.make_weight_bytes(n, k, qtype, seed=n)
        x = synth.make_x(2, k, seed=n)
        ref = O.c_matmul(O.bf16_bits(x), w, qtype)
        check_close(run_fused(x, w, qtype), ref)
        assert O.rel_l2(run_fused(x, w, qtype, torch.float32), ref) <= 2e-5


def test_leading_dims_and_router():
    w = synth.make_weight(128, 512, QT.Q4_K, seed=1)
    x = to_x(synth.make_x(6, 512, seed=1)).reshape(2, 3, 512)
    y = gj.matmul(x, w)
    assert y.shape == (2, 3, 128) and y.dtype == torch.bfloat16
    ref = O.c_matmul(O.bf16_bits(x.reshape(6, 512).float().cpu().numpy()), w.data.cpu().numpy(), QT.Q4_K)
    check_close(y.reshape(6, 128).float().cpu().numpy(), ref)


@pytest.mark.parametrize("qtype", REFERENCE_FUSED, ids=lambda t: t.name)
@pytest.mark.parametrize("m", [1, 8, 64, 512])
def test_dispatch_agrees_with_fallback(qtype, m):
    """matmul (fused where it applies) == dequant_matmul, to the tolerance of the reference's
    tests/test_matmul.py:177-189."""
    w = synth.make_weight(128, 512, qtype, seed=m)
    x = to_x(synth.make_x(m, 512, seed=m))
    got = gj.matmul(x, w).float().cpu().numpy()
    want = gj.dequant_matmul(x, w).float().cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2 * np.abs(want).max())


@pytest.mark.parametrize("m", [1, 4, 512])
def test_dequant_matmul_matches_plain(m):
    w = synth.make_weight(128, 512, QT.Q4_K, seed=m)
    x = to_x(synth.make_x(m, 512, seed=m))
    got = gj.dequant_matmul(x, w).double().cpu().numpy()
    wd = w.dequantize(torch.bfloat16).double().cpu().numpy()
    ref = x.double().cpu().numpy() @ wd.T
    np.testing.assert_allclose(got, ref, rtol=2e-2, atol=2e-2 * np.abs(ref).max())


def test_blocking_does_not_change_the_result():
    w = synth.make_weight(128, 512, QT.Q6_K, seed=3)
    x = to_x(synth.make_x(5, 512, seed=3))
    whole = gj.dequant_matmul(x, w)
    split = gj.dequant_matmul(x, w, block_bytes=4 * 16 * 512)
    assert mm._block_count(128, 512, 4 * 16 * 512) == 8
    assert torch.equal(whole, split)


def test_f32_x_takes_the_fallback():
    w = synth.make_weight(64, 512, QT.Q4_K, seed=9)
    x = torch.from_numpy(synth.make_x(2, 512, seed=9)).cuda()
    y = gj.matmul(x, w)
    assert y.dtype == torch.float32          # promoted, i.e. not the bf16 fused kernel
    with pytest.raises(ValueError):
        kernels.fused_matmul(x, w)


def test_gradient_in_x():
    w = synth.make_weight(64, 512, QT.Q4_K, seed=4)
    for blocks_bytes in (None, 4 * 16 * 512):
        x = to_x(synth.make_x(3, 512, seed=4)).requires_grad_(True)
        y = gj.matmul(x, w, block_bytes=blocks_bytes)
        g = torch.ones_like(y)
        y.backward(g)
        assert x.grad.dtype == x.dtype and x.grad.shape == x.shape
        W = w.dequantize(torch.float32)
        want = (g.float() @ W)
        np.testing.assert_allclose(x.grad.float().cpu().numpy(), want.cpu().numpy(), rtol=2e-2,
                                   atol=2e-2 * float(want.abs().max()))


def test_status_word_is_clean():
    import ctypes
    from gguf_jax_b200 import _lib
    v = ctypes.c_int32(-1)
    assert _lib.lib().ggq_read_status(torch.cuda.current_device(), ctypes.byref(v)) == 0
    assert v.value == 0


# ---- the tuned Q4_K batch-1 kernel (TMA ring + tensor-core dot products + split-K finish) ----

@pytest.mark.parametrize("n,k", [(1, 256), (3, 512), (33, 9 * 256), (200, 11 * 256), (4100, 1024), (20_000, 256),
                                 (8192, 2048), (512, 28672), (1024, 8192), (148 * 32, 4096), (5000, 7 * 256)])
def test_q4k_batch1_kernel_shapes(n, k):
    w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=n + k)
    x = synth.make_x(1, k, seed=n)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)
    got32 = run_fused(x, w, QT.Q4_K, torch.float32)
    assert O.rel_l2(got32, ref) <= 2e-5, (n, k, O.rel_l2(got32, ref))
    got16 = run_fused(x, w, QT.Q4_K)
    assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())
    check_close(got16, ref)


def test_q4k_batch1_kernel_is_deterministic_and_leaves_scratch_clean():
    shapes = [(8192, 2048), (200, 11 * 256), (4100, 1024)]
    first = {}
    for rep in range(3):
        for n, k in shapes:
            w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=1)
            x = synth.make_x(1, k, seed=2)
            got = run_fused(x, w, QT.Q4_K, torch.float32)
            if rep == 0:
                first[(n, k)] = got
                assert O.rel_l2(got, O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)) <= 2e-5
            else:
                assert np.array_equal(got.view(np.uint32), first[(n, k)].view(np.uint32))


def test_q4k_scratch_is_reusable_across_shapes():
    """One scratch buffer serves calls of any shape in any order: a small weight followed by a
    large one (whose arrival counters sit where the small call's partial sums could have gone)."""
    for n, k in [(96, 512), (33, 9 * 256), (4752, 4096), (20_000, 256), (96, 512), (8192, 2048), (4736, 4096)]:
        w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=3)
        x = synth.make_x(1, k, seed=4)
        ref = O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)
        assert O.rel_l2(run_fused(x, w, QT.Q4_K, torch.float32), ref) <= 2e-5, (n, k)


# ---- the tuned Q5_K batch-1 kernel ----

@pytest.mark.parametrize("n,k", [(1, 256), (3, 512), (33, 9 * 256), (200, 11 * 256), (4100, 1024), (20_000, 256),
                                 (512, 28672), (1024, 8192), (148 * 32, 4096), (5000, 7 * 256)])
def test_q5k_batch1_kernel_shapes(n, k):
    w = synth.make_weight_bytes(n, k, QT.Q5_K, seed=n + k)
    x = synth.make_x(1, k, seed=n)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q5_K)
    got32 = run_fused(x, w, QT.Q5_K, torch.float32)
    assert O.rel_l2(got32, ref) <= 2e-5, (n, k, O.rel_l2(got32, ref))
    got16 = run_fused(x, w, QT.Q5_K)
    assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())
    check_close(got16, ref)


def test_q5k_batch1_kernel_one_hot_every_position_of_a_superblock():
    n, k = 40, 768
    w = synth.make_weight_bytes(n, k, QT.Q5_K, seed=78)
    W = O.ref_dequantize(w, QT.Q5_K)
    for col in list(range(256, 512)) + [3, 700]:
        x = np.zeros((1, k), dtype=np.float32)
        x[0, col] = 1.0
        got = run_fused(x, w, QT.Q5_K, torch.float32)
        assert np.array_equal(got[0], W[:, col]), col


def test_q5k_batch1_kernel_is_deterministic():
    first = {}
    for rep in range(3):
        for n, k in [(8192, 2048), (200, 11 * 256), (4100, 1024)]:
            w = synth.make_weight_bytes(n, k, QT.Q5_K, seed=1)
            x = synth.make_x(1, k, seed=2)
            got = run_fused(x, w, QT.Q5_K, torch.float32)
            if rep == 0:
                first[(n, k)] = got
            else:
                assert np.array_equal(got.view(np.uint32), first[(n, k)].view(np.uint32))


# ---- the tuned Q6_K batch-1 kernel (rows must start 16-byte aligned: K a multiple of 2048) ----

@pytest.mark.parametrize("n,k", [(1, 2048), (3, 2048), (33, 4096), (200, 6144), (4100, 2048), (512, 28672),
                                 (1024, 8192), (148 * 32, 4096), (5000, 2048), (32, 2048), (31, 4096)])
def test_q6k_batch1_kernel_shapes(n, k):
    w = synth.make_weight_bytes(n, k, QT.Q6_K, seed=n + k)
    x = synth.make_x(1, k, seed=n)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q6_K)
    got32 = run_fused(x, w, QT.Q6_K, torch.float32)
    assert O.rel_l2(got32, ref) <= 2e-5, (n, k, O.rel_l2(got32, ref))
    got16 = run_fused(x, w, QT.Q6_K)
    assert np.array_equal(got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())
    check_close(got16, ref)


def test_q6k_batch1_kernel_one_hot_every_position_of_a_superblock():
    """x = e_k returns column k of the decoded weight exactly, for every k of one superblock of
    every alignment class (the block's offset in its 16-byte window is 2 j mod 16)."""
    n, k = 40, 2048
    w = synth.make_weight_bytes(n, k, QT.Q6_K, seed=77)
    W = O.ref_dequantize(w, QT.Q6_K)
    for col in list(range(0, 256)) + [256 * j + 31 * j + 5 for j in range(1, 8)]:
        x = np.zeros((1, k), dtype=np.float32)
        x[0, col] = 1.0
        got = run_fused(x, w, QT.Q6_K, torch.float32)
        assert np.array_equal(got[0], W[:, col]), col


def test_q6k_batch1_kernel_is_deterministic_and_shares_scratch_with_q4k():
    first = {}
    for rep in range(3):
        for qt, n, k in [(QT.Q6_K, 8192, 2048), (QT.Q4_K, 4100, 1024), (QT.Q6_K, 200, 6144), (QT.Q6_K, 4736, 4096)]:
            w = synth.make_weight_bytes(n, k, qt, seed=1)
            x = synth.make_x(1, k, seed=2)
            got = run_fused(x, w, qt, torch.float32)
            if rep == 0:
                first[(qt, n, k)] = got
                assert O.rel_l2(got, O.c_matmul(O.bf16_bits(x), w, qt)) <= 2e-5
            else:
                assert np.array_equal(got.view(np.uint32), first[(qt, n, k)].view(np.uint32))


@pytest.mark.parametrize("log2_scale", [-70, -20, 0, 35, 110])
def test_q6k_batch1_kernel_activation_magnitudes(log2_scale):
    n, k = 256, 2048
    w = synth.make_weight_bytes(n, k, QT.Q6_K, seed=8)
    x = synth.make_x(1, k, seed=9) * np.float32(2.0 ** log2_scale)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q6_K)
    got = run_fused(x, w, QT.Q6_K, torch.float32)
    assert np.isfinite(got).all()
    assert O.rel_l2(got, ref) <= 2e-5, O.rel_l2(got, ref)


# ---- the tcgen05 / TMEM kernel for larger batches (tf32 operands, float32 accumulation) ----

GEMM_TYPES = [QT.Q4_K, QT.Q5_K, QT.Q6_K, QT.IQ4_XS, QT.Q8_0, QT.IQ2_XS, QT.Q2_K]


@pytest.fixture(autouse=True)
def _tf32_kernel_for_the_gemm_tests(request, monkeypatch):
    # Q4_K / Q5_K / Q6_K have faster kernels behind ggq_gemm; these tests are about the tf32 one that serves every format
    if request.node.name.startswith("test_tensor_core_gemm"):
        monkeypatch.setenv("GGQ_GEMM_KERNEL", "tf32")


@pytest.mark.parametrize("qtype", GEMM_TYPES, ids=lambda t: t.name)
@pytest.mark.parametrize("m", [17, 32, 100, 128, 200, 256, 300, 512])
def test_tensor_core_gemm_matches_oracle(qtype, m):
    n, k = 200, 11 * 256           # one full and one ragged 128-row tile, 88 K blocks
    w = synth.make_weight_bytes(n, k, qtype, seed=m)
    x = synth.make_x(m, k, seed=m)
    ref = O.c_matmul(O.bf16_bits(x), w, qtype)
    got32 = run_fused(x, w, qtype, torch.float32)
    # tf32 weights (11 significant bits, rounded to nearest): about 3e-4 relative L2
    assert O.rel_l2(got32, ref) <= 1e-3, O.rel_l2(got32, ref)
    check_close(run_fused(x, w, qtype), ref)


@pytest.mark.parametrize("m", [256 + 96, 512 + 88, 512 + 128, 768 + 240])
def test_tensor_core_gemm_narrower_last_batch_tile(m):
    # the last batch tile is narrower than the full ones, holds more stages and needs its own share of shared memory
    # (Q8_0 and IQ4_XS always take the tf32 kernel; Q6_K takes it when its rows are not 16-byte aligned)
    for qtype, n, k in [(QT.Q8_0, 200, 512), (QT.IQ4_XS, 130, 768), (QT.Q6_K, 128, 256)]:
        w = synth.make_weight_bytes(n, k, qtype, seed=m)
        x = synth.make_x(m, k, seed=m)
        ref = O.c_matmul(O.bf16_bits(x), w, qtype)
        assert O.rel_l2(run_fused(x, w, qtype, torch.float32), ref) <= 1e-3


def test_tensor_core_gemm_large_tile_counts():
    for n, k, m in [(1024, 512, 64), (4096, 4096, 32), (130, 256, 20)]:
        w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=n)
        x = synth.make_x(m, k, seed=n)
        ref = O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)
        check_close(run_fused(x, w, QT.Q4_K), ref)


def test_tensor_core_gemm_one_hot_columns():
    """x = e_k returns the weight column: exact up to the tf32 rounding of the weight, i.e. the
    bf16 result is the bf16 rounding of the float32 weight or its neighbour."""
    n, k = 130, 512
    w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=2)
    W = O.ref_dequantize(w, QT.Q4_K)
    cols = list(range(0, 512, 16))
    x = np.zeros((len(cols), k), dtype=np.float32)
    x[np.arange(len(cols)), cols] = 1.0
    got = run_fused(x, w, QT.Q4_K, torch.float32)
    want = W[:, cols].T
    np.testing.assert_allclose(got, want, rtol=2.0 ** -11, atol=0)


def test_tensor_core_gemm_split_k_is_deterministic_and_leaves_scratch_clean():
    """Few row tiles: the launch cuts K into ranges and the last CTA of a tile adds the partial
    tiles.  Same bits every time, and the batch-1 kernel (which shares the counter area of the
    scratch) still works in between."""
    n, k, m = 512, 16 * 256, 48
    w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=21)
    x = synth.make_x(m, k, seed=22)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)
    first = run_fused(x, w, QT.Q4_K, torch.float32)
    assert O.rel_l2(first, ref) <= 1e-3
    x1 = synth.make_x(1, k, seed=23)
    ref1 = O.c_matmul(O.bf16_bits(x1), w, QT.Q4_K)
    for _ in range(3):
        assert O.rel_l2(run_fused(x1, w, QT.Q4_K, torch.float32), ref1) <= 2e-5
        again = run_fused(x, w, QT.Q4_K, torch.float32)
        assert (again.view(np.uint32) == first.view(np.uint32)).all()


def test_router_cap_and_fallback_above_it():
    w = synth.make_weight(256, 512, QT.Q4_K, seed=5)
    cap = gj.fused_batch_limit(w)
    assert cap == kernels.gemv_max_batch()
    for m in (cap, cap + 1):
        x = to_x(synth.make_x(m, 512, seed=5))
        ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), w.data.cpu().numpy(), QT.Q4_K)
        got = gj.matmul(x, w).float().cpu().numpy()
        if m <= cap:
            check_close(got, ref)
        else:   # decode to bf16 + library GEMM: the reference's own tolerance for that route
            np.testing.assert_allclose(got, ref, rtol=2e-2, atol=2e-2 * np.abs(ref).max())


@pytest.mark.parametrize("log2_scale", [-70, -40, -20, 0, 25, 35, 70, 110])
def test_q4k_batch1_kernel_activation_magnitudes(log2_scale):
    """The kernel rescales the activations by a power of two internally; the result must not
    depend on their magnitude (a second staging pass handles tensors far from unit scale)."""
    n, k = 256, 1024
    w = synth.make_weight_bytes(n, k, QT.Q4_K, seed=8)
    x = synth.make_x(1, k, seed=9) * np.float32(2.0 ** log2_scale)
    ref = O.c_matmul(O.bf16_bits(x), w, QT.Q4_K)
    got = run_fused(x, w, QT.Q4_K, torch.float32)
    assert np.isfinite(got).all()
    assert O.rel_l2(got, ref) <= 2e-5, O.rel_l2(got, ref)


def test_q4k_batch1_kernel_zero_activations():
    w = synth.make_weight_bytes(64, 512, QT.Q4_K, seed=1)
    got = run_fused(np.zeros((1, 512), np.float32), w, QT.Q4_K, torch.float32)
    assert (got == 0).all()
