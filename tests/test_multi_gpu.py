"""Row sharding on real GPUs: on every rank the sharded result equals the single-device result
of the same kernels on the whole weight, up to the order in which float32 partial sums of a row
are added (the bound is pinned in multi_gpu_worker.same), for the NCCL all-gather route and for
both in-kernel exchanges (flags and tagged words), eager and replayed from a CUDA graph.  Runs on
2, 4 and 8 ranks as far as the box has GPUs; skipped with fewer than two."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_sharding_matches_single_device(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env, cwd=ROOT)
    assert r.returncode == 0 and f"MULTI_GPU_OK world={world}" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
