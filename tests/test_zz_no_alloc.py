"""The scratch-free Q4_K entry point, ggq_gemv_q4k_static.

It serves callers that may not allocate device memory around a call (a framework's custom-call
handler that only receives operands and results, a serving loop with a fixed memory plan): the partial sums and arrival counters that ggq_gemv keeps in a
caller-provided buffer sit in a device array built into the library instead.  The test drives it
through the C ABI twice in a row -- the second call reuses whatever the first left in the shared
array -- and requires the same float32 result as ggq_gemv, bit for bit (same kernel, same split).
Collected last on purpose, so a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import _lib, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _run(fn_name, w, x, n, k, with_workspace):
    L = _lib.lib()
    y = torch.full((1, n), float("nan"), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    if with_workspace:
        need = L.ggq_workspace_bytes(int(QT.Q4_K), n, k, 1)
        ws = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
        _lib.check(L.ggq_gemv(int(QT.Q4_K), w.data_ptr(), n, k, x.data_ptr(), 1, y.data_ptr(), _lib.GGQ_F32,
                              ws.data_ptr(), ws.numel(), stream))
    else:
        _lib.check(L.ggq_gemv_q4k_static(w.data_ptr(), n, k, x.data_ptr(), y.data_ptr(), _lib.GGQ_F32, stream))
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_static_scratch_entry_point_matches_ggq_gemv_twice_in_a_row():
    for n, k in [(4752, 4096), (200, 11 * 256)]:      # both shapes cut row groups across CTAs
        wb = synth.make_weight_bytes(n, k, QT.Q4_K, seed=5)
        xb = synth.make_x(1, k, seed=6)
        w = torch.from_numpy(wb).cuda()
        x = torch.from_numpy(xb).cuda().to(torch.bfloat16)
        want = _run("ggq_gemv", w, x, n, k, with_workspace=True)
        assert O.rel_l2(want, O.c_matmul(O.bf16_bits(xb), wb, QT.Q4_K)) <= 2e-5
        first = _run("ggq_gemv_q4k_static", w, x, n, k, with_workspace=False)
        second = _run("ggq_gemv_q4k_static", w, x, n, k, with_workspace=False)
        assert np.array_equal(first.view(np.uint32), want.view(np.uint32)), (n, k)
        assert np.array_equal(second.view(np.uint32), want.view(np.uint32)), (n, k)


def test_static_scratch_entry_point_rejects_what_it_cannot_hold():
    L = _lib.lib()
    w = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1024, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(16, dtype=torch.float32, device="cuda")
    rc = L.ggq_gemv_q4k_static(w.data_ptr(), 524288 + 1, 256, x.data_ptr(), y.data_ptr(), _lib.GGQ_F32, None)
    assert rc == 2 and b"524288" in L.ggq_last_error()
    rc = L.ggq_gemv_q4k_static(w.data_ptr(), 8, 100, x.data_ptr(), y.data_ptr(), _lib.GGQ_F32, None)
    assert rc == 2
