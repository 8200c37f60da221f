#!/usr/bin/env python
"""Headline benchmark: fused Q4_K GEMV on an 8192 x 28672 weight at batch 1.

One *step* is one fused multiply ``y = x @ W.T`` of a bf16 activation row against one
Q4_K weight (132 MB of blocks).  Steps rotate over several distinct weight copies whose
total size is a multiple of the 126 MB L2, so every step streams its weight from HBM.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 (launched under torchrun, one rank per GPU): the weight's output rows are sharded
across the ranks, every rank multiplies its slice and the kernel's epilogue stores the rows
into every rank's output over NVLink (NCCL all-gather if symmetric memory is unavailable)
-- total work is fixed, so scaling is "strong".

Rank 0 prints ONE JSON line.  Keys beyond the common contract:
  roofline     achieved = algorithmic bytes of one launch / mean launch time (CUDA events
               around the timed region, on the launching stream); peak = measured copy
               bandwidth from MEASURED_PEAKS.json (fallback 6650 GB/s, marked as such).
  cpu_baseline the CPU restatement of the same multiply (oracle/, OpenMP) timed on this
               host on a bounded row sample of the same weight.
  decode       tokens/s of a Llama-3-70B-shaped Q4_K_M decode step at batch 1 (the second half
               of the headline metric): per layer five fused GEMVs -- q+k (Q4_K 9216x8192),
               v (Q6_K 1024x8192), o (Q4_K 8192x8192), gate+up (Q4_K 57344x8192), down (Q6_K
               8192x28672) -- 80 layers, then the Q6_K lm_head 128256x8192; every GEMV is
               row-sharded over the N ranks.  Norms, RoPE, attention and sampling are outside the
               reference and are not run: each GEMV reads a fixed synthetic activation vector.
  e2e          the same multiply through the public API (gguf_jax_b200.matmul) with the
               activation coming from pinned host memory and the result read back to the
               host inside the timed region; the weight stays resident on the device, as in
               the reference, where parameters live on the device and only activations move.

``--impl reference`` times the reference's CPU route (dequantize + multiply, restated in
oracle/ because JAX is not installed here) with all host threads on a bounded row sample
per step, and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS, K_DIM, BATCH = 8192, 28672, 1
QTYPE_NAME = "Q4_K"
METRIC = "q4_k_fused_gemv_hbm_throughput"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from
# the ncu capture summarised under profiles/ (None until captured).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 134_400_000
NCU_TRAFFIC_SOURCE = ("profiles/q4k_gemv_m1_8192x28672.md (dram__bytes_read.sum + dram__bytes_write.sum of the kernel with TMA boxes, mean of "
                      "three launches of one ncu metrics capture, 1 GPU, full weight)")


def algorithmic_bytes(n: int, k: int, m: int, out_itemsize: int = 2) -> int:
    """Quantized weight + activations + output: the bytes one launch must move."""
    return n * (k // 256) * 144 + 2 * m * k + out_itemsize * m * n


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback (6650 GB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 100 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                p = [s.strip() for s in line.split(",")]
                if len(p) < 9:
                    continue
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                for name, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:  # noqa: BLE001
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_product(min_seconds: float, min_passes: int, warmup: int) -> dict:
    """Times the CPU restatement of the reference's route (dequantize + multiply, fused per row, float32,
    oracle/, OpenMP) on the whole 8192 x 28672 weight of the headline workload with every host core.
    Used by both the ``cpu_baseline`` key and ``--impl reference``, so the two always agree on code path,
    sample and thread count.  The thread count is set explicitly: launchers such as torchrun export
    OMP_NUM_THREADS=1 to their children."""
    from gguf.constants import GGMLQuantizationType as QT

    from gguf_jax_b200 import synth
    from oracle import oracle as O

    cores = O.set_threads(os.cpu_count() or 1)
    qt = QT[QTYPE_NAME]
    w = synth.make_weight_bytes(N_ROWS, K_DIM, qt, seed=0)
    x = O.bf16_bits(synth.make_x(BATCH, K_DIM, seed=0))
    for _ in range(max(1, warmup)):
        O.c_matmul(x, w, qt, plain_f32=True)
    # the timed region is `min_passes` passes; it is repeated whole until `min_seconds` have gone by
    t0 = time.perf_counter()
    passes = 0
    while True:
        for _ in range(min_passes):
            O.c_matmul(x, w, qt, plain_f32=True)
        passes += min_passes
        dt = time.perf_counter() - t0
        if dt >= min_seconds or dt >= 120.0:
            break
    per_pass = algorithmic_bytes(N_ROWS, K_DIM, BATCH, 4)
    return {"value": per_pass * passes / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "passes": passes, "seconds": dt,
            "sample": f"{passes} passes over all {N_ROWS} rows of the Q4_K weight (K={K_DIM}, batch {BATCH}) in "
                      f"{dt:.1f} s; CPU restatement of dequantize + multiply (oracle/, fused per row, float32, "
                      f"OpenMP x{cores}) because JAX is not installed on this image"}


def cpu_baseline() -> dict:
    out = cpu_product(min_seconds=10.0, min_passes=3, warmup=1)
    return {k: out[k] for k in ("value", "unit", "cores", "kind", "sample")}


# Llama-3-70B-shaped Q4_K_M decode step: (name, qtype, rows, K) of the fused GEMVs of one layer.
DECODE_LAYER = [("qk", "Q4_K", 9216, 8192), ("v", "Q6_K", 1024, 8192), ("o", "Q4_K", 8192, 8192),
                ("gate_up", "Q4_K", 57344, 8192), ("down", "Q6_K", 8192, 28672)]
DECODE_HEAD = ("lm_head", "Q6_K", 128256, 8192)
DECODE_LAYERS = 80
DECODE_DISTINCT = 8      # distinct layer weight sets cycled through the 80 layer steps
_BLOCK_BYTES = {"Q4_K": 144, "Q6_K": 210}


def _scale_block_scales(w, log2: int) -> None:
    """Multiply the float16 super-block scales of a Q4_K / Q6_K payload by 2^log2 in place (exact)."""
    import torch
    ts = _BLOCK_BYTES[w.qtype.name]
    blocks = w.data.view(-1, ts)
    cols = slice(0, 4) if w.qtype.name == "Q4_K" else slice(208, 210)
    f = blocks[:, cols].contiguous().view(torch.float16)
    blocks[:, cols] = (f.float() * (2.0 ** log2)).to(torch.float16).view(torch.uint8)


def decode_leg(world: int, rank: int, dev, batch: int = 1, route: str = "fused") -> dict:
    """Time one decode step of the 70B-shaped model at `batch` sequences; see the module docstring.

    The GEMVs are chained for real: q+k and v read the previous layer's down output, o reads the
    first 8192 outputs of q+k, gate+up reads o, down reads the first 28672 outputs of gate+up, the
    lm_head reads the last down output.  (Attention, norms and activations are not run, so the
    numbers mean nothing; the block scales are shifted by powers of two beforehand so that the
    magnitudes stay near one along the chain.)  On N > 1 ranks every product is row-sharded and
    its result reaches every rank through an exchange inside the kernels: tagged words at batch 1,
    peer stores plus one flag per launch for larger batches.
    `route` "fused" calls the fused kernels by name (above the small-batch cap that is the tcgen05
    code GEMM); "router" calls `matmul`, which above the cap decodes and calls the library GEMM."""
    import torch
    import torch.distributed as dist
    from gguf.constants import GGMLQuantizationType as QT

    import gguf_jax_b200 as gj
    from gguf_jax_b200 import kernels, sharded, synth

    def shard(qt_name, rows, k, seed):
        qt = QT[qt_name]
        rows_local = rows // world
        assert rows_local * world == rows
        # the same model at every N: a matrix is drawn whole from a seed that names only the matrix,
        # then this rank keeps its row range (what a row-sliced upload of a model file would hold)
        w = synth.make_weight_on_device(rows, k, qt, seed=seed, device=dev)
        mine = w.data[rank * rows_local:(rank + 1) * rows_local].clone()
        del w
        return gj.QuantizedArray(mine, qt, (rows_local, k))

    layers = [[shard(q, n, k, 100 + 10 * li + i) for i, (_, q, n, k) in enumerate(DECODE_LAYER)]
              for li in range(DECODE_DISTINCT)]
    head = shard(DECODE_HEAD[1], DECODE_HEAD[2], DECODE_HEAD[3], 999)
    launches = DECODE_LAYERS * len(DECODE_LAYER) + 1
    x0 = torch.from_numpy(synth.make_x(batch, 8192, seed=8192)).to(dev).to(torch.bfloat16)
    product = kernels.fused_matmul if route == "fused" else gj.matmul

    if batch > 1 and world > 1:
        # the batch-major kernel stores this rank's columns of every batch row into every rank's buffer and raises a flag
        # (ggq_gemm_sharded); a product may read the leading columns of a buffer two launches back, hence four buffers
        po = sharded.PeerOutput(None, max_batch=batch, n_total=DECODE_HEAD[2], device=dev, n_buffers=4)

        def mm(x, w):
            return po.matmul(x[:, :w.shape[1]], w, wait_previous=True)

        def value(h):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            return h.clone()
    elif batch > 1:
        def mm(x, w):
            return product(x[:, :w.shape[1]].contiguous(), w)

        def value(h):
            return h
    elif world > 1:
        ex = sharded.TaggedExchange(None, n_max=DECODE_HEAD[2], device=dev,
                                    n_buffers=sharded.TaggedExchange.buffers_for(launches, max_back=2))

        def mm(x, w):
            return ex.matmul(x, w)

        def value(h):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            return h.to_tensor().clone()
    else:
        def mm(x, w):
            return kernels.fused_matmul(x[:, :w.shape[1]], w)

        def value(h):
            return h

    def layer_step(h, ws):
        qk = mm(h, ws[0])
        mm(h, ws[1])                 # v: consumed by attention, which is not run
        o = mm(qk, ws[2])
        gu = mm(o, ws[3])
        return mm(gu, ws[4])

    # calibration: shift every matrix's block scales so that its output has rms ~ 1 for an rms ~ 1 input
    def calibrate(x, w):
        y = value(mm(x, w)).float()
        rms = float(y.pow(2).mean().sqrt())
        sh = -int(round(__import__("math").log2(rms))) if rms > 0 and rms == rms else 0
        _scale_block_scales(w, sh)
        return (y * 2.0 ** sh).to(torch.bfloat16)

    h = x0
    for ws in layers:
        qk = calibrate(h, ws[0])
        calibrate(h, ws[1])
        o = calibrate(qk[:, :8192].contiguous(), ws[2])
        gu = calibrate(o, ws[3])
        h = calibrate(gu[:, :28672].contiguous(), ws[4])
    calibrate(h, head)

    last_hidden = [None]

    def token():
        h = x0
        for li in range(DECODE_LAYERS):
            h = layer_step(h, layers[li % DECODE_DISTINCT])
        last_hidden[0] = h
        return mm(h, head)

    import ctypes

    from gguf_jax_b200 import _lib

    def device_status() -> int:
        word = ctypes.c_int32(0)
        _lib.lib().ggq_read_status(dev.index, ctypes.byref(word))
        return int(word.value)

    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        t0 = time.perf_counter()
        logits = token()
        stream.synchronize()
        eager_s = time.perf_counter() - t0
        # a bounded wait that ran out (a peer's words never arrived) shows here: do not go on to
        # replay hundreds of launches that would each sit out their wait limit
        bad = torch.tensor([1 if (device_status() != 0 or eager_s > 20.0) else 0], device=dev)
        if world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            raise RuntimeError(f"decode chain gave up after its first token: device status {device_status()}, "
                               f"{eager_s:.1f} s for one eager token")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            logits = token()
    torch.cuda.synchronize()

    def one() -> float:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(3):
        one()
    ms = statistics.median([one() for _ in range(10)])
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    lv = value(logits).float()
    finite = bool(torch.isfinite(lv).all())
    # parity along the chain: every product of the first layer step and the lm_head, each fed with the
    # vector the chain itself produced, on sampled rows of this rank's shard against the CPU checker.
    # The logits themselves are NOT comparable between N to the last place: the chain is linear and
    # unnormalised (80 products of non-normal random matrices), so the last-place differences of a
    # different split order grow to per cents of a common scale factor by the end; the checksum is
    # there to show that, not to be matched.
    import numpy as np
    from oracle import oracle as O

    def product_error(x_full, w, y_full, n_pick, seed):
        rows_local = w.shape[0]
        pick = np.sort(np.random.default_rng(seed).choice(rows_local, size=min(n_pick, rows_local), replace=False))
        w_rows = w.data[torch.from_numpy(pick).to(dev)].cpu().numpy()
        xin = x_full.float().reshape(batch, -1)[:, :w.shape[1]].cpu().numpy()
        ref = O.c_matmul(O.bf16_bits(xin), w_rows, w.qtype)
        got = y_full.float().reshape(batch, -1)[:, rank * rows_local + torch.from_numpy(pick).to(dev)].cpu().numpy()
        return O.rel_l2(got, ref)

    errs = [product_error(value(last_hidden[0]), head, lv, 128, 7)]
    ws0 = layers[0]
    h0 = x0
    qk = value(mm(x0, ws0[0]))
    errs.append(product_error(h0, ws0[0], qk, 128, 11))
    vv = value(mm(x0, ws0[1]))
    errs.append(product_error(h0, ws0[1], vv, 128, 12))
    qk_h = mm(x0, ws0[0])
    o_h = mm(qk_h, ws0[2])
    o_v = value(o_h)
    gu_h = mm(o_h, ws0[3])
    gu_v = value(gu_h)
    d_v = value(mm(gu_h, ws0[4]))
    errs.append(product_error(qk, ws0[2], o_v, 128, 13))
    errs.append(product_error(o_v, ws0[3], gu_v, 128, 14))
    errs.append(product_error(gu_v, ws0[4], d_v, 128, 15))
    head_err = torch.tensor([errs[0], max(errs)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(head_err, op=dist.ReduceOp.MAX)
    checksum = {"logits_abs_mean": float(lv.abs().mean()), "logits_sum": float(lv.double().sum()),
                "logits_first8": [float(v) for v in lv.reshape(-1)[:8]]}
    wbytes = sum(n * (k // 256) * _BLOCK_BYTES[q] for _, q, n, k in DECODE_LAYER) * DECODE_LAYERS
    wbytes += DECODE_HEAD[2] * (DECODE_HEAD[3] // 256) * _BLOCK_BYTES[DECODE_HEAD[1]]
    del graph
    exchange = "none" if world == 1 else (
        "stored into every rank's buffer by the batch-major kernel, one flag per launch (ggq_gemm_sharded)" if batch > 1 else
        "tagged words stored into every rank's buffer by the kernels (ggq_gemv_sharded_tagged)")
    return {"tok_s": batch * 1e3 / ms, "ms_per_token": ms / batch, "ms_per_step": ms, "batch": batch, "route": route, "launches_per_step": launches,
            "weight_gb_per_step": wbytes / 1e9, "aggregate_hbm_gbs": wbytes / (ms * 1e-3) / 1e9,
            "logits_finite": finite, "logits_rms": float(lv.pow(2).mean().sqrt()), "device_status": device_status(),
            "parity": {"lm_head_rel_l2_vs_oracle": float(head_err[0].item()),
                       "worst_of_first_layer_and_head_rel_l2_vs_oracle": float(head_err[1].item()),
                       "rows": 6 * 128 * world, "bar": 3e-3,
                       "note": "each product fed with the vector the chain produced; sampled rows of every rank's shard"},
            "checksum": checksum,
            "exchange": exchange,
            "model": "Llama-3-70B-shaped Q4_K_M (attn_v, ffn_down, lm_head in Q6_K), GEMVs only, chained",
            "note": f"{DECODE_LAYERS} layer steps cycle over {DECODE_DISTINCT} distinct synthetic layer weight sets "
                    "(each far larger than L2); block scales shifted by powers of two so the chain stays near unit "
                    "magnitude; one CUDA graph per token"}


# ---------------------------------------------------------------------------------------------
# Other configurations of the workload family, measured on one GPU next to the headline (own keys in
# the JSON line, outside the headline's timed region).

LOWBIT_SWEEP = ["Q2_K", "IQ1_S", "IQ1_M", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ4_XS"]
LLAMA_1B_LAYER = [("q", "Q4_K", 2048, 2048), ("k", "Q4_K", 512, 2048), ("v", "Q6_K", 512, 2048), ("o", "Q4_K", 2048, 2048),
                  ("gate", "Q4_K", 8192, 2048), ("up", "Q4_K", 8192, 2048), ("down", "Q6_K", 2048, 8192)]
LLAMA_8B_SHAPES = [("attn_q", "Q5_K", 4096, 4096), ("attn_k", "Q5_K", 1024, 4096), ("ffn_gate", "Q6_K", 14336, 4096),
                   ("ffn_down", "Q6_K", 4096, 14336)]


def _graph_us(calls, repeats: int = 5) -> float:
    """Median microseconds per call of a list of zero-argument launches, replayed as one CUDA graph."""
    import torch
    for f in calls:
        f()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for f in calls:
                f()
    ts = []
    for _ in range(repeats + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(st):
            e0.record(st)
            g.replay()
            e1.record(st)
        st.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / len(calls))
    del g
    return float(statistics.median(ts[1:]))


def extra_legs(dev) -> dict:
    import numpy as np
    import torch
    from gguf.constants import GGML_QUANT_SIZES
    from gguf.constants import GGMLQuantizationType as QT

    import gguf_jax_b200 as gj
    from gguf_jax_b200 import kernels, synth
    from oracle import oracle as O

    peak, _ = measured_peak()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f)["bf16_tflops_sustained"])
    except Exception:  # noqa: BLE001
        tf_peak = 1400.0

    def wbytes(qt, n, k):
        bs, ts = GGML_QUANT_SIZES[qt]
        return n * (k // bs) * ts

    def x_of(m, k, seed=0):
        return torch.from_numpy(synth.make_x(m, k, seed=seed)).to(dev).to(torch.bfloat16)

    def sampled_parity(x, w, y, rows=64):
        pick = np.sort(np.random.default_rng(3).choice(w.shape[0], size=min(rows, w.shape[0]), replace=False))
        ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), w.data[torch.from_numpy(pick).to(dev)].cpu().numpy(), w.qtype)
        return O.rel_l2(y.float()[:, torch.from_numpy(pick).to(dev)].cpu().numpy(), ref)

    out = {}

    # ---- the low-bit sweep: nine qtypes on 8192 x 28672 at batch 1, 4, 8
    sweep = {}
    for name in LOWBIT_SWEEP:
        qt = QT[name]
        nbytes = wbytes(qt, N_ROWS, K_DIM)
        copies = max(3, -(-300_000_000 // nbytes))
        ws = [synth.make_weight_on_device(N_ROWS, K_DIM, qt, seed=40 + c, device=dev) for c in range(copies)]
        row = {}
        for m in (1, 4, 8):
            x = x_of(m, K_DIM, m)
            us = _graph_us([(lambda w=w: kernels.fused_matmul(x, w)) for w in ws * 2])
            moved = nbytes + 2 * m * K_DIM + 2 * m * N_ROWS
            row[f"m{m}"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_measured_hbm": moved / us / 1e3 / peak}
        x = x_of(4, K_DIM, 4)
        row["rel_l2_sampled_rows_m4"] = sampled_parity(x, ws[0], kernels.fused_matmul(x, ws[0], out_dtype=torch.float32))
        sweep[name] = row
        del ws
        torch.cuda.empty_cache()
    out["lowbit_sweep_8192x28672"] = sweep

    # ---- Llama-3.2-1B-shaped decode layer (Q4_K with attn_v / ffn_down in Q6_K), a 16-layer stack per batch
    layers = [[synth.make_weight_on_device(n, k, QT[q], seed=1000 + 10 * li + i, device=dev)
               for i, (_, q, n, k) in enumerate(LLAMA_1B_LAYER)] for li in range(16)]
    layer_bytes = sum(wbytes(QT[q], n, k) for _, q, n, k in LLAMA_1B_LAYER)
    stack = {}
    for m in (1, 2, 4, 8, 16):
        xs = {k: x_of(m, k, m) for k in (2048, 8192)}
        calls = [(lambda w=w: kernels.fused_matmul(xs[w.shape[1]], w)) for ws in layers for w in ws]
        us_layer = _graph_us(calls) * len(LLAMA_1B_LAYER)
        moved = layer_bytes + sum(2 * m * (n + k) for _, _, n, k in LLAMA_1B_LAYER)
        stack[f"m{m}"] = {"us_per_layer": us_layer, "gbs": moved / us_layer / 1e3, "frac_of_measured_hbm": moved / us_layer / 1e3 / peak}
    x = x_of(4, 8192, 4)
    stack["rel_l2_sampled_rows_down_m4"] = sampled_parity(x, layers[0][6], kernels.fused_matmul(x, layers[0][6], out_dtype=torch.float32))
    stack["layer_bytes"] = layer_bytes
    stack["note"] = "16 distinct layers (621 MB) in one CUDA graph, seven fused launches per layer"
    out["llama_1b_layer_q4_k_m"] = stack
    del layers
    torch.cuda.empty_cache()

    # ---- Llama-3-8B shapes in Q5_K / Q6_K through the public matmul at 1, 32, 128, 512 tokens (the router picks the route)
    shapes = {}
    for tag, q, n, k in LLAMA_8B_SHAPES:
        qt = QT[q]
        nbytes = wbytes(qt, n, k)
        copies = max(3, -(-300_000_000 // nbytes))
        ws = [synth.make_weight_on_device(n, k, qt, seed=70 + c, device=dev) for c in range(copies)]
        cap = gj.fused_batch_limit(ws[0])
        row = {"fused_batch_limit": cap}
        for m in (1, 32, 128, 512):
            x = x_of(m, k, m)
            us = _graph_us([(lambda w=w: gj.matmul(x, w)) for w in ws * 2], repeats=3)
            moved = nbytes + 2 * m * k + 2 * m * n
            flops = 2.0 * m * n * k
            row[f"m{m}"] = {"us": us, "route": "fused" if m <= cap else "decode kernel + library GEMM", "gbs": moved / us / 1e3,
                            "tflops": flops / us / 1e6, "frac_of_measured_hbm": moved / us / 1e3 / peak,
                            "frac_of_sustained_bf16": flops / us / 1e6 / tf_peak}
        x = x_of(32, k, 32)
        row["rel_l2_sampled_rows_m32"] = sampled_parity(x, ws[0], gj.matmul(x, ws[0]))     # bf16 output: ~1.6e-3 is its rounding
        shapes[f"{tag}_{q}_{n}x{k}"] = row
        del ws
        torch.cuda.empty_cache()
    out["llama_8b_shapes"] = shapes

    # ---- the decode kernel: bytes in + bytes out per second
    dec = {}
    for q in ("Q4_K", "Q6_K", "IQ4_XS", "IQ2_XS"):
        qt = QT[q]
        n, k = 16384, 8192
        ws = [synth.make_weight_on_device(n, k, qt, seed=90 + c, device=dev) for c in range(3)]
        for dt, item in ((torch.bfloat16, 2), (torch.float32, 4)):
            us = _graph_us([(lambda w=w: w.dequantize(dt)) for w in ws * 2], repeats=3)
            moved = wbytes(qt, n, k) + n * k * item
            dec[f"{q}_{'bf16' if item == 2 else 'f32'}"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_measured_hbm": moved / us / 1e3 / peak}
        del ws
        torch.cuda.empty_cache()
    out["dequantize_16384x8192"] = dec

    # ---- the reference's own CPU-runnable case: Q4_K 4096 x 4096, decode bit-exact and fused product at batch 1
    qt = QT["Q4_K"]
    n = k = 4096
    wb = synth.make_weight_bytes(n, k, qt, seed=4096)
    ws = [gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device=dev)] + \
         [synth.make_weight_on_device(n, k, qt, seed=4097 + c, device=dev) for c in range(31)]       # 32 x 9.4 MB > 2 x L2
    x = x_of(1, k, 1)
    dense = ws[0].dequantize(torch.float32).cpu().numpy()
    ref_dense = O.c_dequantize(wb, qt)
    us = _graph_us([(lambda w=w: gj.matmul(x, w)) for w in ws * 2])
    y = gj.matmul(x, ws[0]).float().cpu().numpy()
    ref = O.c_matmul(O.bf16_bits(x.float().cpu().numpy()), wb, qt)
    moved = wbytes(qt, n, k) + 2 * k + 2 * n
    out["q4_k_4096x4096_m1"] = {"us": us, "gbs": moved / us / 1e3, "frac_of_measured_hbm": moved / us / 1e3 / peak,
                                "decode_bit_exact": bool((dense.view(np.uint32) == ref_dense.view(np.uint32)).all()),
                                "rel_l2_all_rows": O.rel_l2(y, ref)}
    return out


def check_headline(world, rank, dev, qt, weights, x, step, y_local, use_peer, y_full) -> dict:
    """Outside the timed region: run the timed step once more for each weight copy and compare what it
    left behind (the whole gathered output on every rank) with the CPU checker on sampled rows of this
    rank's shard and, on N > 1 ranks, with the one-GPU kernel on the whole weight."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import gguf_jax_b200 as gj
    from gguf_jax_b200 import kernels, synth
    from oracle import oracle as O

    rows_local = N_ROWS // world
    worst_oracle, worst_single, exact_min, n_rows = 0.0, 0.0, 1.0, 0
    xb = O.bf16_bits(x.float().cpu().numpy())
    for c in range(len(weights)):
        step(c)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        y = y_local[0]
        if use_peer:
            full = y.to_tensor().float().reshape(-1)
        elif world > 1:
            full = y_full.float().reshape(-1)
        else:
            full = y.float().reshape(-1)
        pick = np.random.default_rng(100 + c).choice(rows_local, size=48, replace=False)
        pick.sort()
        w_rows = weights[c].data[torch.from_numpy(pick).to(dev)].cpu().numpy()
        ref = O.c_matmul(xb, w_rows, qt).reshape(-1)
        got = full[rank * rows_local + torch.from_numpy(pick).to(dev)].cpu().numpy()
        worst_oracle = max(worst_oracle, O.rel_l2(got, ref))
        n_rows += len(pick)
        if world > 1:
            whole = synth.make_weight_on_device(N_ROWS, K_DIM, qt, seed=c, device=dev)
            single = kernels.fused_matmul(x, whole).float().reshape(-1)
            del whole
            exact_min = min(exact_min, float((single == full).float().mean()))
            worst_single = max(worst_single, float((single - full).norm() / single.norm()))
    if world > 1:
        t = torch.tensor([worst_oracle, worst_single, -exact_min], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst_oracle, worst_single, exact_min = float(t[0]), float(t[1]), -float(t[2])
    # The output is bf16: rounding alone (unit roundoff 2^-8) gives a relative L2 error of 1.6e-3 to 2.2e-3 on a sample
    # of 48 values, 3.9e-3 at the very worst; the kernel's own float32 arithmetic is five orders below that.
    out = {"rows": n_rows * world, "rel_l2": worst_oracle, "bar": 3e-3,
           "against": "oracle c_matmul (double accumulation) on 48 sampled rows per rank and weight copy; the error is "
                      "the rounding of the bf16 output"}
    if world > 1:
        out["vs_one_gpu_kernel"] = {"rel_l2": worst_single, "identical_fraction": exact_min,
                                    "note": "whole gathered output of every rank against ggq_gemv on the full weight"}
    if not worst_oracle <= 3e-3:
        raise RuntimeError(f"headline output fails parity: {out}")
    return out


def run_reference(args) -> None:
    """--impl reference: the CPU route on this host's cores; rank 0 only.  One step = one product over the
    whole weight; at least ``--steps`` of them and at least two seconds are timed."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    out = cpu_product(min_seconds=2.0, min_passes=max(1, args.steps), warmup=max(1, min(args.warmup, 3)))
    value = out["value"]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": max(1, args.steps), "warmup": max(1, min(args.warmup, 3)), "ms_per_step": out["seconds"] / out["passes"] * 1e3,
        "timed_regions": out["passes"] // max(1, args.steps),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (numpy default_rng blocks, f16 super-scales |N(0,1)|*2^-7)",
        "config": {"workload": f"Q4_K fused GEMV {N_ROWS}x{K_DIM} batch {BATCH}", "rows": N_ROWS},
        "cpu_baseline": {k: out[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from gguf.constants import GGMLQuantizationType as QT

    import gguf_jax_b200 as gj
    from gguf_jax_b200 import _lib, kernels, sharded, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()
    if args.profile and (args.profile_shape or args.profile_batch != BATCH or args.profile_qtype not in ("Q4_K", "Q5_K", "Q6_K")):
        # any format, shape and batch through the public product: three distinct weights in turn
        n_rows, k_dim = (int(v) for v in (args.profile_shape or f"{N_ROWS}x{K_DIM}").lower().split("x"))
        qt = QT[args.profile_qtype]
        ws = [synth.make_weight_on_device(n_rows, k_dim, qt, seed=c, device=dev) for c in range(3)]
        xp = torch.from_numpy(synth.make_x(args.profile_batch, k_dim, seed=0)).to(dev).to(torch.bfloat16)
        for i in range(args.warmup + args.steps):
            kernels.fused_matmul(xp, ws[i % 3])
        torch.cuda.synchronize()
        print(f"profile run: {args.warmup + args.steps} eager launches of {qt.name} {n_rows}x{k_dim} batch "
              f"{args.profile_batch} done", file=sys.stderr)
        return
    qt = QT[args.profile_qtype if args.profile else QTYPE_NAME]

    rows_local = N_ROWS // world
    assert rows_local * world == N_ROWS
    copies = 4  # 4 x 132 MB = 528 MB of distinct weights, > 4x the 126 MB L2
    weights = []
    for c in range(copies):
        full = synth.make_weight_on_device(N_ROWS, K_DIM, qt, seed=c, device=dev)
        shard = full.data[rank * rows_local:(rank + 1) * rows_local].contiguous()
        weights.append(gj.QuantizedArray(shard, qt, (rows_local, K_DIM)))
        del full
    x = torch.from_numpy(synth.make_x(BATCH, K_DIM, seed=0)).to(dev).to(torch.bfloat16)
    y_local = [None]
    y_full = torch.empty((world, BATCH, rows_local), dtype=torch.bfloat16, device=dev) if world > 1 else None

    # N > 1: the kernel itself pushes its rows into every rank's output buffer over NVLink and
    # raises a flag; the next launch waits for all flags (ggq_gemv_sharded).  NCCL all-gather is
    # the fallback if symmetric memory cannot be set up.
    peer = None
    exchange = "none"
    if world > 1:
        try:
            peer = sharded.TaggedExchange(None, n_max=N_ROWS, device=dev,
                                          n_buffers=sharded.TaggedExchange.buffers_for(args.steps, max_back=1))
            exchange = ("tagged words stored into every rank's buffer by the kernel; each launch waits until the "
                        "previous exchange has landed (ggq_gemv_sharded_tagged)")
        except Exception as e:  # noqa: BLE001
            exchange = f"NCCL all-gather (symmetric memory unavailable: {type(e).__name__})"
            if rank == 0:
                print(f"[bench] {exchange}: {e}", file=sys.stderr)
    prev = [None]          # the previous step's result: the next launch is ordered after it
    seam = [False]         # first launch of a captured graph: its predecessor is not in the graph

    use_peer = [peer is not None]

    def step(i: int):
        if use_peer[0]:
            y = peer.matmul(x, weights[i % copies], after=None if (seam[0] and i == 0) else prev[0])
            prev[0] = y
        else:
            y = kernels.fused_matmul(x, weights[i % copies])
            if world > 1:
                dist.all_gather_into_tensor(y_full, y)
        y_local[0] = y

    if args.profile:
        for i in range(args.warmup + args.steps):
            step(i)
        torch.cuda.synchronize()
        print(f"profile run: {args.warmup + args.steps} eager launches done", file=sys.stderr)
        if world > 1:
            dist.barrier()
            sys.stderr.flush()
            os._exit(0)
        return

    stream = torch.cuda.Stream(dev)
    launches_per_step = 1
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i)
        stream.synchronize()
        if world > 1 and use_peer[0]:
            # a flag wait that ran out during the warm-up means the peers' stores do not arrive:
            # fall back to the NCCL route rather than sit out the wait limit on every step
            import ctypes
            word = ctypes.c_int32(0)
            _lib.lib().ggq_read_status(dev.index, ctypes.byref(word))
            bad = torch.tensor([1 if word.value else 0], device=dev)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if int(bad.item()):
                use_peer[0] = False
                exchange = "NCCL all-gather (the fused exchange's bounded wait expired during warm-up)"
                for i in range(3):
                    step(i)
                stream.synchronize()
        # one CUDA graph of `steps` launches: the Python/ctypes launch cost would otherwise
        # exceed the ~20 us kernel
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            seam[0] = True
            with torch.cuda.graph(graph, stream=stream):
                for i in range(args.steps):
                    step(i)
            seam[0] = False
        except Exception as e:  # noqa: BLE001
            graph = None
            if rank == 0:
                print(f"[bench] graph capture unavailable ({type(e).__name__}: {e}); timing eager launches",
                      file=sys.stderr)
    torch.cuda.synchronize()

    def timed_region() -> float:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            if graph is not None:
                graph.replay()
            else:
                for i in range(args.steps):
                    step(i)
            e1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    warm_ms = timed_region()  # one untimed replay so the graph itself is warm
    # Repeat the timed region for about a second so the clock sampler sees the load.  The count
    # is decided on rank 0 and shared: every rank must replay the same number of times (the fused
    # exchange and the barriers are collective).
    # (~3 s: nvidia-smi needs a few hundred ms before its first sample)
    repeats = max(3, min(3000, int(3000.0 / max(warm_ms, 0.01))))
    if world > 1:
        t = torch.tensor([repeats], device=dev)
        dist.broadcast(t, 0)
        repeats = int(t.item())
    with ClockSampler(local_rank) as clocks:
        ms_all = [timed_region() for _ in range(repeats)]
    ms = ms_all[0]
    clk = clocks.summary()
    ms = statistics.median(ms_all)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    parity = check_headline(world, rank, dev, qt, weights, x, step, y_local, use_peer[0], y_full)

    total_bytes = algorithmic_bytes(N_ROWS, K_DIM, BATCH) * args.steps
    value = total_bytes / (ms * 1e-3) / 1e9
    launch_bytes = algorithmic_bytes(rows_local, K_DIM, BATCH)
    launch_ms = ms / args.steps
    peak, peak_src = measured_peak()
    achieved = launch_bytes / (launch_ms * 1e-3) / 1e9

    # end to end through the public API: activation from pinned host memory, result to host
    xh = x.cpu().pin_memory()
    yh = torch.empty((BATCH, N_ROWS), dtype=torch.bfloat16).pin_memory()
    e2e_steps = min(args.steps, 200)

    def e2e_step(i: int):
        if world > 1:
            xd = xh.to(dev, non_blocking=True)
            # the public sharded call: local fused product, then the all-gather, all stream-ordered (the
            # in-kernel exchange orders launches against each other, not against a host read-back)
            y = gj.matmul(xd, weights[i % copies])
            dist.all_gather_into_tensor(y_full, y)
            yh.view(world, BATCH, rows_local).copy_(y_full, non_blocking=True)
        else:
            # one GPU: the public call takes the pinned host tensors themselves - the activations are fetched by a
            # small kernel in front of the product (ggq_stage_host) and the product stores into the pinned result
            gj.matmul(xh, weights[i % copies], out=yh)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = algorithmic_bytes(N_ROWS, K_DIM, BATCH) * e2e_steps / e2e_s / 1e9
    if world == 1:
        # what the last step left in the host buffer is the device-resident product, bit for bit
        want = kernels.fused_matmul(x, weights[(e2e_steps - 1) % copies]).cpu()
        if not torch.equal(yh, want):
            raise RuntimeError("end-to-end leg: the host result differs from the device-resident product")

    decode = None
    if not args.no_decode:
        # free the headline weights first: the decode leg brings its own
        weights.clear()
        torch.cuda.empty_cache()
        try:
            decode = decode_leg(world, rank, dev)
        except Exception as e:  # noqa: BLE001
            decode = {"unavailable": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()
        # the same step at 32 sequences: above the small-batch cap, so the fused route is the tcgen05
        # code GEMM called by name; on one GPU the router's route (decode + library GEMM) is timed beside it
        try:
            decode["batch32"] = decode_leg(world, rank, dev, batch=32, route="fused")
            torch.cuda.empty_cache()
            if world == 1:
                decode["batch32_router"] = decode_leg(world, rank, dev, batch=32, route="router")
                torch.cuda.empty_cache()
        except Exception as e:  # noqa: BLE001
            decode["batch32"] = {"unavailable": f"{type(e).__name__}: {e}"}

    legs = None
    if world == 1 and not args.no_legs:
        try:
            legs = extra_legs(dev)
        except Exception as e:  # noqa: BLE001
            legs = {"unavailable": f"{type(e).__name__}: {e}"}

    if rank == 0:
        cpu = cpu_baseline() if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": launch_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (every block byte uniform random, f16 super-scales |N(0,1)|*2^-7: the seeded recipe of "
                    "the shape's config, drawn with the device generator instead of numpy default_rng because the "
                    "weights are generated in place on the GPU)",
            "config": {
                "workload": f"Q4_K fused GEMV {N_ROWS}x{K_DIM} batch {BATCH} (bf16 x, bf16 y)",
                "rows_per_gpu": rows_local, "parallelism": f"row-sharded x{world}; exchange: {exchange}" if world > 1 else "1 GPU",
                "l2_policy": f"inputs larger than L2: steps rotate over {copies} distinct weights "
                             f"({copies * algorithmic_bytes(N_ROWS, K_DIM, 0) / 1e6:.0f} MB)",
                "timing": "CUDA events around one CUDA graph of all steps" if graph is not None else "CUDA events around eager launches",
                "repeats": len(ms_all),
            },
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "peak_source": peak_src,
                "traffic": (NCU_TRAFFIC_BYTES_PER_LAUNCH * rows_local // N_ROWS) if NCU_TRAFFIC_BYTES_PER_LAUNCH else None,
                "traffic_source": NCU_TRAFFIC_SOURCE + ("" if world == 1 else
                                                         "; scaled by rows_per_gpu / 8192, not captured on a shard (every weight "
                                                         "row is read once, so traffic grows in proportion to the rows)"),
                "algorithmic_bytes_per_launch": launch_bytes, "launch_us": launch_ms * 1e3,
            },
            "clocks": clk,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * BATCH * K_DIM,
                    "d2h_bytes_per_step": 2 * BATCH * N_ROWS, "steps": e2e_steps,
                    "ms_per_step": e2e_s / e2e_steps * 1e3,
                    "note": ("weight resident on the device; every step gguf_jax_b200.matmul(x_pinned, w, out=y_pinned): the activations "
                             "are fetched from pinned host memory by a kernel in front of the product, the product stores its result "
                             "into pinned host memory, then the stream is synchronised; the last result is checked against the "
                             "device-resident product bit for bit") if world == 1 else
                            "weight resident on the device; activation H2D from pinned memory, fused product on the shard, "
                            "NCCL all-gather and result D2H every step, then the stream is synchronised"},
            "gpu_launches": args.steps * launches_per_step,
            "parity": parity,
        }
        if decode is not None:
            line["decode"] = decode
        if legs is not None:
            line["legs"] = legs
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)       # out of the process before any tear-down
    if world > 1:
        # Tear down without destroy_process_group(): with NCCL kernels captured in a CUDA graph it
        # has been seen to block at exit.  Everything is flushed and every rank has passed the
        # barrier, so a plain process exit is safe.
        del graph
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-qtype", default=QTYPE_NAME,
                    choices=["Q4_K", "Q5_K", "Q6_K", "Q2_K", "IQ4_XS", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S",
                             "IQ1_S", "IQ1_M"],
                    help="with --profile: the qtype of the weight")
    ap.add_argument("--profile-shape", default="", help="with --profile: ROWSxCOLS of the weight (default 8192x28672)")
    ap.add_argument("--profile-batch", type=int, default=BATCH, help="with --profile: rows of x (default 1)")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-step (tokens/s) leg")
    ap.add_argument("--no-legs", action="store_true", help="skip the one-GPU legs for the other configurations")
    ap.add_argument("--profile", action="store_true",
                    help="profiler-friendly run: a few eager launches of the hot kernel, no graph, "
                         "no CPU baseline, no end-to-end leg, no JSON line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
