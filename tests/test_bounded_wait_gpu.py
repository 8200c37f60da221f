"""A bounded device-side wait that runs out must come back by itself, raise the status word once,
and leave the device usable.  One GPU, no peer, no fault: the kernel behind
ggq_gemv_sharded_tagged is told that its activations are tagged words of an earlier exchange and
is pointed at a zero-filled local buffer; tag 0 is never valid, so every poll fails until the wait's
time limit (about 50 ms) passes, the launch finishes on whatever it read, and ggq_read_status
reports GGQ_TIMEOUT.  The flag protocol's wait (ggq_gemv_sharded with wait_previous) is expired
the same way: world = 2 with both "peers" local and the second rank's flag never raised.
"""
import ctypes

import numpy as np
import pytest
import torch
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import _lib, kernels, synth
from gguf_jax_b200.array import QuantizedArray
from oracle import oracle as O

pytestmark = pytest.mark.gpu
GGQ_TIMEOUT = 6


def _status(L):
    word = ctypes.c_int32(-1)
    rc = L.ggq_read_status(torch.cuda.current_device(), ctypes.byref(word))
    return rc, word.value


def _plain_product_is_still_right(n, k):
    wb = synth.make_weight_bytes(n, k, QT.Q4_K, seed=3)
    xb = synth.make_x(1, k, seed=4)
    w = QuantizedArray.from_bytes(wb, QT.Q4_K, shape=(n, k), device="cuda")
    y = kernels.fused_matmul(torch.from_numpy(xb).cuda().to(torch.bfloat16), w, out_dtype=torch.float32)
    assert O.rel_l2(y.cpu().numpy(), O.c_matmul(O.bf16_bits(xb), wb, QT.Q4_K)) <= 2e-5


def test_tagged_wait_runs_out_and_reports_timeout():
    L = _lib.lib()
    dev = torch.cuda.current_device()
    assert L.ggq_init(dev) == 0
    assert _status(L) == (0, 0)
    n, k = 32, 256                       # one CTA, one superblock: a single wait expires
    w = torch.from_numpy(synth.make_weight_bytes(n, k, QT.Q4_K, seed=1)).cuda()
    x_tagged = torch.zeros(k, dtype=torch.int32, device="cuda")          # tag 0: never valid
    y = torch.zeros(n, dtype=torch.int32, device="cuda")
    state = torch.zeros(64, dtype=torch.int32, device="cuda")
    ws = torch.zeros(max(L.ggq_workspace_bytes(int(QT.Q4_K), n, k, 1), 256), dtype=torch.uint8, device="cuda")
    peers = (ctypes.c_void_p * 1)(y.data_ptr())
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.check(L.ggq_gemv_sharded_tagged(int(QT.Q4_K), w.data_ptr(), n, k, None, x_tagged.data_ptr(), 1, None, 0, 0,
                                         peers, state.data_ptr(), 1, 0, n, ws.data_ptr(), ws.numel(),
                                         torch.cuda.current_stream().cuda_stream))
    t1.record()
    torch.cuda.synchronize()
    assert 20.0 <= t0.elapsed_time(t1) <= 2000.0       # the wait ran for its limit and then returned
    rc, word = _status(L)
    assert rc == GGQ_TIMEOUT and word & 1
    assert b"bounded" in L.ggq_last_error()
    assert _status(L) == (0, 0)                         # reading clears it
    assert int(state[1].item()) == 1                    # the launch still completed its bookkeeping
    _plain_product_is_still_right(200, 1024)
    assert _status(L) == (0, 0)


def test_flag_wait_runs_out_and_reports_timeout():
    L = _lib.lib()
    n, k = 32, 256
    w = torch.from_numpy(synth.make_weight_bytes(n, k, QT.Q4_K, seed=2)).cuda()
    x = torch.from_numpy(synth.make_x(1, k, seed=2)).cuda().to(torch.bfloat16)
    y0 = torch.zeros(2 * n, dtype=torch.bfloat16, device="cuda")
    y1 = torch.zeros(2 * n, dtype=torch.bfloat16, device="cuda")
    f0 = torch.zeros(64, dtype=torch.int32, device="cuda")        # rank 0's flags: slot 1 is never raised
    f1 = torch.zeros(64, dtype=torch.int32, device="cuda")        # stands for rank 1's flag array
    ws = torch.zeros(max(L.ggq_workspace_bytes(int(QT.Q4_K), n, k, 1), 256), dtype=torch.uint8, device="cuda")
    ys = (ctypes.c_void_p * 2)(y0.data_ptr(), y1.data_ptr())
    fs = (ctypes.c_void_p * 2)(f0.data_ptr(), f1.data_ptr())
    st = torch.cuda.current_stream().cuda_stream

    def launch(wait):
        _lib.check(L.ggq_gemv_sharded(int(QT.Q4_K), w.data_ptr(), n, k, x.data_ptr(), 1, ys, fs, 2, 0, 2 * n, _lib.GGQ_BF16,
                                      wait, ws.data_ptr(), ws.numel(), st))

    launch(0)                          # exchange 1 published by "rank 0" only
    torch.cuda.synchronize()
    assert _status(L) == (0, 0)
    assert f0[0].item() == 1 and f1[0].item() == 1 and f0[1].item() == 0
    launch(1)                          # waits for rank 1's flag of exchange 1, which never comes
    torch.cuda.synchronize()
    rc, word = _status(L)
    assert rc == GGQ_TIMEOUT and word & 1
    assert _status(L) == (0, 0)
    # rows 0..n-1 of both outputs were still written by the launch that gave up
    ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), w.cpu().numpy(), QT.Q4_K)
    np.testing.assert_allclose(y1[:n].float().cpu().numpy().reshape(1, n), ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
    _plain_product_is_still_right(64, 512)
