"""The per-format operand builders of the tiled fused multiply (gguf_jax_b200/csrc/tile_formats.cuh)
are plain host/device code; this test compiles them for the host and checks, on random blocks,
that every lane run / octet reproduces the decoded weights bit for bit: codes, signs, the
activation map, the scale of every group and the offset terms.  CPU only."""
import os
import subprocess

import numpy as np
import pytest
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import _lib, synth
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "tile_formats_check.cpp")
TILE_QTYPES = [QT.Q4_K, QT.Q5_K, QT.Q6_K, QT.Q2_K, QT.IQ4_XS, QT.IQ2_XXS, QT.IQ2_XS, QT.IQ2_S, QT.IQ3_XXS, QT.IQ3_S, QT.IQ1_S, QT.IQ1_M]
_TAB_OFFSET = {QT.IQ2_XXS: (0, 2048), QT.IQ2_XS: (2048, 4096), QT.IQ2_S: (6144, 8192), QT.IQ3_XXS: (14336, 1024),
               QT.IQ3_S: (15360, 2048), QT.IQ1_S: (17408, 16384), QT.IQ1_M: (17408, 16384)}


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("native") / "tile_formats_check")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.run([cxx, "-O1", "-std=c++17", "-ffp-contract=off", "-o", exe, SRC], check=True, capture_output=True)
    return exe


def kernel_table(qtype) -> bytes:
    """The lookup table as the kernel holds it in shared memory."""
    blob = _lib.tables_blob()
    if qtype == QT.IQ4_XS:
        kv = blob[33792:33808].view(np.int8).astype(np.int16) + 128
        return kv.astype(np.uint8).tobytes()
    if qtype not in _TAB_OFFSET:
        return b"\0" * 16
    off, size = _TAB_OFFSET[qtype]
    t = blob[off:off + size]
    if qtype in (QT.IQ1_S, QT.IQ1_M):
        t = (8 * t.view(np.int8).astype(np.int16) + 9).astype(np.uint8)     # codes 8 * grid + 9
    return t.tobytes()


@pytest.mark.parametrize("qtype", TILE_QTYPES, ids=lambda t: t.name)
def test_operands_reproduce_the_decoded_weights(qtype, checker, tmp_path):
    n_blocks = 96
    blocks = synth.random_blocks(qtype, n_blocks, seed=int(qtype))
    dense = O.c_dequantize(blocks, qtype).astype(np.float32)
    O.assert_bitwise_equal(dense, O.ref_dequantize(blocks, qtype), qtype.name)
    (tmp_path / "b.bin").write_bytes(blocks.tobytes())
    (tmp_path / "d.bin").write_bytes(dense.tobytes())
    (tmp_path / "t.bin").write_bytes(kernel_table(qtype))
    r = subprocess.run([checker, str(int(qtype)), str(tmp_path / "b.bin"), str(tmp_path / "d.bin"), str(tmp_path / "t.bin"),
                        str(n_blocks)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 mismatches" in r.stdout
