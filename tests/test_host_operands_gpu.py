"""Activations and results in pinned host memory (``ggq_stage_host`` in front of the product, the product's stores
going straight to the host buffer) against the same product with device tensors: bit for bit the same result."""
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import kernels, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qtype,n,k,m", [(QT.Q4_K, 512, 4096, 1), (QT.Q6_K, 300, 2048, 1), (QT.Q5_K, 256, 2048, 1),
                                          (QT.IQ4_XS, 128, 2048, 4), (QT.Q4_K, 4096, 6144, 12), (QT.Q8_0, 64, 512, 3)],
                         ids=lambda v: getattr(v, "name", str(v)))
def test_pinned_activations_and_result_match_device_tensors(qtype, n, k, m):
    w = synth.make_weight_on_device(n, k, qtype, seed=3, device="cuda")
    x = torch.from_numpy(synth.make_x(m, k, seed=4)).to(torch.bfloat16)
    want = gj.matmul(x.cuda(), w)
    xh = x.pin_memory()
    # pinned activations, device result
    got = gj.matmul(xh, w)
    assert got.is_cuda and torch.equal(got, want)
    # pinned activations, pinned result; twice on different data, so that a stale staging buffer would show
    yh = torch.zeros((m, n), dtype=torch.bfloat16).pin_memory()
    back = gj.matmul(xh, w, out=yh)
    torch.cuda.synchronize()
    assert back.data_ptr() == yh.data_ptr() and torch.equal(yh, want.cpu())
    x2 = (x * 0.5).pin_memory()
    gj.matmul(x2, w, out=yh)
    torch.cuda.synchronize()
    assert torch.equal(yh, gj.matmul(x2.cuda(), w).cpu())
    # device activations, pinned float32 result
    yf = torch.zeros((m, n), dtype=torch.float32).pin_memory()
    kernels.fused_matmul(x.cuda(), w, out=yf)
    torch.cuda.synchronize()
    assert torch.equal(yf, kernels.fused_matmul(x.cuda(), w, out_dtype=torch.float32).cpu())


def test_host_operand_errors():
    w = synth.make_weight_on_device(64, 512, QT.Q4_K, seed=1, device="cuda")
    x = torch.zeros((1, 512), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="pageable"):
        gj.matmul(x, w)                                  # not pinned
    with pytest.raises(RuntimeError, match="pageable"):
        gj.matmul(x.cuda(), w, out=torch.zeros((1, 64), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="shape"):
        gj.matmul(x.cuda(), w, out=torch.zeros((1, 65), dtype=torch.bfloat16).pin_memory())
    with pytest.raises(ValueError):
        gj.matmul(x.float().pin_memory(), w)             # float32 activations take the materializing route: device only
    big = torch.zeros((64, 512), dtype=torch.bfloat16).cuda()
    with pytest.raises(ValueError, match="batch rows"):
        kernels.fused_matmul(big, w, out=torch.zeros((64, 64), dtype=torch.bfloat16).pin_memory())
