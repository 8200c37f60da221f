"""Seeded synthetic quantized weights and activations.

No GGUF model file ships with this repository, so benchmarks and tests draw block data
from a seed: every byte uniform random, then the f16 super-block scales overwritten with
small finite values so products stay finite.  This is the reference's own test fixture
recipe (tests/test_matmul.py:25-48 there) extended to every block qtype.
"""
from __future__ import annotations

import numpy as np
import torch
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

from .array import QuantizedArray

# byte offsets of the f16 super-scales inside a block: qtype -> (offset, how many f16)
_SCALE_AT = {
    QT.Q4_K: (0, 2), QT.Q5_K: (0, 2), QT.Q6_K: (208, 1), QT.Q2_K: (80, 2), QT.Q3_K: (108, 1),
    QT.IQ4_XS: (0, 1), QT.IQ2_XXS: (0, 1), QT.IQ2_XS: (0, 1), QT.IQ2_S: (0, 1), QT.IQ3_XXS: (0, 1),
    QT.IQ3_S: (0, 1), QT.IQ1_S: (0, 1), QT.Q4_0: (0, 1), QT.Q5_0: (0, 1), QT.Q8_0: (0, 1),
    QT.IQ4_NL: (0, 1), QT.Q4_1: (0, 2), QT.Q5_1: (0, 2), QT.TQ1_0: (52, 1), QT.TQ2_0: (64, 1),
}

BLOCK_QTYPES = tuple(sorted((*_SCALE_AT.keys(), QT.IQ1_M, QT.MXFP4, QT.NVFP4), key=lambda t: t.name))


def random_blocks(qtype: QT, n_blocks: int, seed: int = 0, finite: bool = True) -> np.ndarray:
    """``uint8[n_blocks, type_size]``.  ``finite=False`` leaves every byte random
    (non-finite f16 scales included), the decode-exactness fixture."""
    rng = np.random.default_rng(seed)
    ts = GGML_QUANT_SIZES[qtype][1]
    data = rng.integers(0, 256, size=(n_blocks, ts), dtype=np.uint8)
    if not finite:
        return data
    if qtype in _SCALE_AT:
        off, cnt = _SCALE_AT[qtype]
        scale = (np.abs(rng.normal(size=(n_blocks, cnt))) * 2.0 ** -7).astype(np.float16)
        data[:, off:off + 2 * cnt] = scale.view(np.uint8)
    elif qtype == QT.IQ1_M:
        # the f16 scale is spread over the top nibbles of the four u16 words at bytes 48..55
        bits = (np.abs(rng.normal(size=n_blocks)) * 2.0 ** -7).astype(np.float16).view(np.uint16)
        words = data[:, 48:56].copy().view(np.uint16)
        for j in range(4):
            words[:, j] = (words[:, j] & 0x0FFF) | (((bits >> (4 * j)) & 0xF) << 12)
        data[:, 48:56] = words.view(np.uint8)
    elif qtype == QT.MXFP4:
        data[:, 0] = rng.integers(112, 128, size=n_blocks, dtype=np.uint8)  # scale 2^-16 .. 2^-1
    # NVFP4: every UE4M3 scale byte decodes to a finite value
    return data


def make_weight_bytes(n: int, k: int, qtype: QT, seed: int = 0) -> np.ndarray:
    """Row-major payload ``uint8[n, k // block * type_size]`` of an (n, k) weight."""
    bs, ts = GGML_QUANT_SIZES[qtype]
    if k % bs:
        raise ValueError(f"k={k} is not a multiple of the {qtype.name} block of {bs}")
    return random_blocks(qtype, n * (k // bs), seed).reshape(n, (k // bs) * ts)


def make_weight(n: int, k: int, qtype: QT, seed: int = 0, device=None) -> QuantizedArray:
    return QuantizedArray.from_bytes(make_weight_bytes(n, k, qtype, seed), qtype, shape=(n, k), device=device)


def make_weight_on_device(n: int, k: int, qtype: QT, seed: int, device) -> QuantizedArray:
    """Same distribution drawn with the device's generator: for weights too large to
    stage through the host (tens of GB).  Not bit-identical to :func:`make_weight`."""
    bs, ts = GGML_QUANT_SIZES[qtype]
    nb = n * (k // bs)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    data = torch.randint(0, 256, (nb, ts), dtype=torch.uint8, device=device, generator=g)
    if qtype in _SCALE_AT:
        off, cnt = _SCALE_AT[qtype]
        sc = (torch.randn((nb, cnt), device=device, generator=g).abs() * 2.0 ** -7).to(torch.float16)
        data[:, off:off + 2 * cnt] = sc.view(torch.uint8)
    elif qtype == QT.MXFP4:
        data[:, 0] = torch.randint(112, 128, (nb,), dtype=torch.uint8, device=device, generator=g)
    elif qtype == QT.IQ1_M:
        bits = (torch.randn(nb, device=device, generator=g).abs() * 2.0 ** -7).to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
        words = data[:, 48:56].contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        for j in range(4):
            words[:, j] = (words[:, j] & 0x0FFF) | (((bits >> (4 * j)) & 0xF) << 12)
        data[:, 48:56] = words.to(torch.int16).view(torch.uint8)
    return QuantizedArray.from_bytes(data.reshape(n, -1), qtype, shape=(n, k), device=device)


def make_x(m: int, k: int, seed: int = 0) -> np.ndarray:
    """Activations: N(0, 1) rounded to bfloat16, returned as float32 (exactly bf16-valued)."""
    x = np.random.default_rng(seed + 10_000).normal(size=(m, k)).astype(np.float32)
    u = x.view(np.uint32)
    u = (u + (((u >> 16) & 1) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)
