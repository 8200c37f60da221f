"""Regenerates tests/golden/decode_golden.npz.

For every decodable block qtype: a few blocks of seeded random bytes (one set fully random,
non-finite scales included, one set with small finite scales) and the float32 bit patterns
``gguf.quants.dequantize`` (gguf 0.19.0) produces for them.  The reference defines
correctness of its decoders as bitwise equality with exactly this function
(tests/test_bitwise.py:65-101 of gguf-jax), and keeps no stored vectors of its own, so
these fixtures pin the procedure + seed.

Also stores, for one small (N, K) weight per fused qtype, the float32 product
``x @ dequantize(w).T`` computed by numpy in float64 and rounded once (the
``dequant_matmul`` of src/gguf_jax/_matmul.py:195-201 at float32 precision).

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import gguf  # noqa: E402
from gguf.constants import GGML_QUANT_SIZES  # noqa: E402

from gguf_jax_b200 import synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_golden.npz")


def main():
    arrays = {}
    with np.errstate(all="ignore"):
        for qt in synth.BLOCK_QTYPES:
            bs, ts = GGML_QUANT_SIZES[qt]
            nb = 3 * max(1, 256 // bs)
            rnd = synth.random_blocks(qt, nb, seed=1000 + int(qt), finite=False)
            fin = synth.random_blocks(qt, nb, seed=2000 + int(qt), finite=True)
            for tag, data in (("rnd", rnd), ("fin", fin)):
                ref = gguf.quants.dequantize(data, qt)
                arrays[f"{qt.name}.{tag}.bytes"] = data
                arrays[f"{qt.name}.{tag}.f32bits"] = ref.view(np.uint32)
            # matmul golden: N=8 rows, K=512, M=3
            k = 512
            w = synth.make_weight_bytes(8, k, qt, seed=3000 + int(qt))
            x = synth.make_x(3, k, seed=int(qt))
            W = gguf.quants.dequantize(w, qt).astype(np.float64)
            y = (x.astype(np.float64) @ W.T).astype(np.float32)
            arrays[f"{qt.name}.mm.w"] = w
            arrays[f"{qt.name}.mm.x"] = x
            arrays[f"{qt.name}.mm.y"] = y
    np.savez_compressed(OUT, **arrays)
    print(OUT, os.path.getsize(OUT), "bytes", len(arrays), "arrays")


if __name__ == "__main__":
    main()
