"""The public `matmul` on the benchmark configurations' own weight shapes and batches, sampled rows
against the CPU oracle: the Llama-3.2-1B-shaped layer (Q4_K with attn_v / ffn_down in Q6_K) at batch
1, 2, 4, 8, 16, and the Llama-3-8B-shaped Q5_K / Q6_K weights at batch 1, 32 and 128 through the
router (above its cap it decodes on the device and calls the library GEMM) and through the fused kernels by name.
Bar: relative L2 <= 2e-3 on the bf16 output where the weights are not rounded (up to 32 rows), 4e-3 where they are
rounded to bf16 first (the reference's contract for its GEMM and its fallback), and the reference's elementwise
rtol = 1e-2, atol = 1e-2 max|ref|."""
import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import kernels, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

LAYER_1B = [("q", QT.Q4_K, 2048, 2048), ("k", QT.Q4_K, 512, 2048), ("v", QT.Q6_K, 512, 2048),
            ("gate", QT.Q4_K, 8192, 2048), ("down", QT.Q6_K, 2048, 8192)]
SHAPES_8B = [("q", QT.Q5_K, 4096, 4096), ("k", QT.Q5_K, 1024, 4096), ("gate", QT.Q6_K, 14336, 4096),
             ("down", QT.Q6_K, 4096, 14336)]


def check(product, name, qt, n, k, m):
    rows = max(48, -(-768 // m))          # enough bf16 outputs for the L2 figure to be a statistic
    w = synth.make_weight_on_device(n, k, qt, seed=n + k, device="cuda")
    x = torch.from_numpy(synth.make_x(m, k, seed=m)).cuda().to(torch.bfloat16)
    y = product(x, w)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    pick = np.sort(np.random.default_rng(n).choice(n, size=min(rows, n), replace=False))
    idx = torch.from_numpy(pick).cuda()
    ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), w.data[idx].cpu().numpy(), qt)
    got = y.float()[:, idx].cpu().numpy()
    # up to 32 rows every fused kernel multiplies exact codes; above, both the fused tensor-core kernel and the fallback
    # (decode to bf16 + library GEMM) round the weights to bf16 first, as the reference's own GEMM and fallback do:
    # twice the bar
    exact = m <= 32 and (product is not gj.matmul or m <= gj.fused_batch_limit(w))
    assert O.rel_l2(got, ref) <= (2e-3 if exact else 4e-3), (name, qt.name, n, k, m)
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_llama_1b_layer_shapes(m):
    for name, qt, n, k in LAYER_1B:
        check(gj.matmul, name, qt, n, k, m)


@pytest.mark.parametrize("m", [1, 32, 128])
def test_llama_8b_shapes_through_the_router(m):
    for name, qt, n, k in SHAPES_8B:
        check(gj.matmul, name, qt, n, k, m)


@pytest.mark.parametrize("m", [32, 128])
def test_llama_8b_shapes_fused_tensor_core_kernel(m):
    for name, qt, n, k in SHAPES_8B:
        check(kernels.fused_matmul, name, qt, n, k, m)
