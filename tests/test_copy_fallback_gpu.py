"""The batch-1 kernels with their weight tiles copied by per-lane cp.async instead of TMA boxes (what they do where the
driver offers no tensor-map encoder).  The switch is read once per process, so the check runs in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import numpy as np, torch
from gguf.constants import GGMLQuantizationType as QT
import gguf_jax_b200 as gj
from gguf_jax_b200 import kernels, synth
from oracle import oracle as O
for qt, shapes in ((QT.Q4_K, [(200, 2816), (512, 28672), (1100, 4096)]), (QT.Q5_K, [(200, 2816), (300, 8192)]),
                   (QT.Q6_K, [(200, 2048), (1024, 8192), (96, 4096)])):
    for n, k in shapes:
        wb = synth.make_weight_bytes(n, k, qt, seed=n)
        w = gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device="cuda")
        x = synth.make_x(1, k, seed=k)
        got = kernels.fused_matmul(torch.from_numpy(x).cuda().to(torch.bfloat16), w, out_dtype=torch.float32).cpu().numpy()
        err = O.rel_l2(got, O.c_matmul(O.bf16_bits(x), wb, qt))
        assert err <= 2e-5, (qt.name, n, k, err)
print("FALLBACK_OK")
"""


def test_cp_async_copy_path_matches_the_oracle():
    env = dict(os.environ, GGQ_Q4K_TMA="0", GGQ_Q5K_TMA="0", GGQ_Q6K_TMA="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FALLBACK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
