"""Worker for tests/test_multi_gpu.py: one process per GPU (launched with torchrun).

Checks, on every rank, that the row-sharded product equals the single-device product of the whole
weight computed by the same kernel -- through the NCCL all-gather route and through the fused
peer-store route (ggq_gemv_sharded) -- and the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from gguf.constants import GGMLQuantizationType as QT  # noqa: E402

import gguf_jax_b200 as gj  # noqa: E402
from gguf_jax_b200 import kernels, sharded, synth  # noqa: E402
from oracle import oracle as O  # noqa: E402


def same(a, b, what):
    """Sharded against unsharded result of the same kernel.  Not bitwise in general: where the K
    range of a row is cut between CTAs depends on how many rows the launch has, so the float32
    partial sums of a row may be added in a different order in a launch over N/P rows than in a
    launch over N rows.  The pinned bound: float32 sums differ by a few ulps, so after the single
    bf16 rounding at most 2 % of the outputs may differ, each by one place (2^-7 relative)."""
    a, b = a.float(), b.float()
    exact = (a == b).float().mean().item()
    assert exact >= 0.98, f"{what}: only {exact:.3f} of the outputs identical"
    assert torch.allclose(a, b, rtol=2.0 ** -7, atol=1e-6 * float(b.abs().max())), what


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    n, k = 1024 * world, 2048
    for qt, m in ((QT.Q4_K, 1), (QT.Q6_K, 4)):
        wb = synth.make_weight_bytes(n, k, qt, seed=11)
        xb = synth.make_x(m, k, seed=12)
        w = gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device=dev)
        x = torch.from_numpy(xb).to(dev).to(torch.bfloat16)
        single = kernels.fused_matmul(x, w)
        shard = sharded.shard_rows(w, rank, world)
        y = sharded.sharded_matmul(x, shard)
        same(y, single, f"rank {rank}: all-gather route ({qt.name})")
        ref = O.c_matmul(O.bf16_bits(xb), wb, qt)
        assert O.rel_l2(y.float().cpu().numpy(), ref) <= 2e-3
    # fused peer-store exchange (batch 1): chained launches of the three tuned kernels reuse both buffers
    m = 1
    out = sharded.PeerOutput(None, max_batch=1, n_total=n, device=dev)
    for step, qt in enumerate((QT.Q4_K, QT.Q6_K, QT.Q5_K, QT.Q4_K, QT.Q6_K)):
        wb = synth.make_weight_bytes(n, k, qt, seed=20 + step)
        xb = synth.make_x(m, k, seed=30 + step)
        w = gj.QuantizedArray.from_bytes(wb, qt, shape=(n, k), device=dev)
        x = torch.from_numpy(xb).to(dev).to(torch.bfloat16)
        single = kernels.fused_matmul(x, w)
        y = out.matmul(x, sharded.shard_rows(w, rank, world), wait_previous=True)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        same(y, single, f"rank {rank}: fused exchange, step {step}")
    # flag exchange, chained: the output of exchange i (written by every rank into every rank's
    # buffer while the consumer kernel may already be resident) is the activation of launch i + 1
    nk = 2048
    fchain = [QT.Q4_K, QT.Q6_K, QT.Q5_K, QT.Q4_K, QT.Q6_K, QT.Q4_K]
    f_full = [gj.QuantizedArray.from_bytes(synth.make_weight_bytes(nk, nk, qt, seed=60 + i), qt, shape=(nk, nk), device=dev)
              for i, qt in enumerate(fchain)]
    f_shards = [sharded.shard_rows(w, rank, world) for w in f_full]
    fout = sharded.PeerOutput(None, max_batch=1, n_total=nk, device=dev, n_buffers=len(fchain))
    fx0 = torch.from_numpy(synth.make_x(1, nk, seed=61)).to(dev).to(torch.bfloat16)

    def run_flag_chain():
        ys, cur = [], fx0
        for i, sh in enumerate(f_shards):
            cur = fout.matmul(cur, sh, wait_previous=i > 0)
            ys.append(cur)
        return ys

    def check_flag_chain(ys, what):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        vals = [y.clone() for y in ys]
        for i, w in enumerate(f_full):
            single = kernels.fused_matmul(fx0 if i == 0 else vals[i - 1], w)
            same(vals[i], single, f"rank {rank}: flag chain {what}, launch {i}")
        dist.barrier()

    check_flag_chain(run_flag_chain(), "eager")
    fst = torch.cuda.Stream(dev)
    with torch.cuda.stream(fst):
        fg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fg, stream=fst):
            f_outs = run_flag_chain()
    for rep in range(2):
        with torch.cuda.stream(fst):
            fg.replay()
        fst.synchronize()
        check_flag_chain(f_outs, f"graph replay {rep}")

    # flag exchange with a batch (ggq_gemm_sharded, batch-major kernel): a chain of products of 12 and of 40 rows (two slices),
    # one of which reads only the leading columns of its predecessor's buffer (row stride larger than K, no copy)
    os.environ["GGQ_GEMM_KERNEL"] = "wide"       # the one-GPU reference above 32 rows: the same exact kernel, not the bf16-weight GEMM
    bk = 2048
    bshapes = [(QT.Q4_K, 4096, bk), (QT.Q6_K, 2048, 2048), (QT.Q5_K, 2048, 2048), (QT.Q6_K, 2048, 2048)]   # (qtype, rows, K)
    b_full = [gj.QuantizedArray.from_bytes(synth.make_weight_bytes(nn, kk, qt, seed=80 + i), qt, shape=(nn, kk), device=dev)
              for i, (qt, nn, kk) in enumerate(bshapes)]
    b_shards = [sharded.shard_rows(w, rank, world) for w in b_full]
    keep = []            # nothing symmetric is freed while a later iteration captures a graph
    for mb in (12, 40):
        bout = sharded.PeerOutput(None, max_batch=mb, n_total=4096, device=dev, n_buffers=len(bshapes))
        bx0 = torch.from_numpy(synth.make_x(mb, bk, seed=81)).to(dev).to(torch.bfloat16)

        def run_batch_chain():
            ys, cur = [], bx0
            for i, sh in enumerate(b_shards):
                cur = bout.matmul(cur[:, :sh.shape[1]], sh, wait_previous=i > 0)      # launch 1 reads 2048 of 4096 columns
                ys.append(cur)
            return ys

        def check_batch_chain(ys, what):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            vals = [y.clone() for y in ys]
            for i, w in enumerate(b_full):
                xin = bx0 if i == 0 else vals[i - 1][:, :w.shape[1]].contiguous()
                same(vals[i], kernels.fused_matmul(xin, w), f"rank {rank}: batch {mb} flag chain {what}, launch {i}")
            dist.barrier()

        check_batch_chain(run_batch_chain(), "eager")
        bst = torch.cuda.Stream(dev)
        with torch.cuda.stream(bst):
            bg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(bg, stream=bst):
                b_outs = run_batch_chain()
        for rep in range(2):
            with torch.cuda.stream(bst):
                bg.replay()
            bst.synchronize()
            check_batch_chain(b_outs, f"graph replay {rep}")
        keep.append((bout, bg, b_outs, run_batch_chain, check_batch_chain))
    del os.environ["GGQ_GEMM_KERNEL"]

    # tagged exchange: a chain whose products feed each other (n = k), including a result consumed
    # two launches later, then the same chain captured in a CUDA graph and replayed
    chain = [QT.Q4_K, QT.Q6_K, QT.Q5_K, QT.Q6_K, QT.Q4_K]
    ws_full = [gj.QuantizedArray.from_bytes(synth.make_weight_bytes(nk, nk, qt, seed=40 + i), qt, shape=(nk, nk), device=dev)
               for i, qt in enumerate(chain)]
    shards = [sharded.shard_rows(w, rank, world) for w in ws_full]
    ex = sharded.TaggedExchange(None, n_max=nk, device=dev, n_buffers=sharded.TaggedExchange.buffers_for(len(chain)))
    x0 = torch.from_numpy(synth.make_x(1, nk, seed=50)).to(dev).to(torch.bfloat16)

    def run_chain():
        outs = [ex.matmul(x0, shards[0])]
        outs.append(ex.matmul(outs[0], shards[1]))
        outs.append(ex.matmul(outs[1], shards[2]))
        outs.append(ex.matmul(outs[1], shards[3]))      # consumes a result two launches old
        outs.append(ex.matmul(outs[3], shards[4], after=outs[2]))   # and ordered after another result
        return outs

    def check_chain(outs, what):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        vals = [o.to_tensor().clone() for o in outs]
        inputs = [x0, vals[0], vals[1], vals[1], vals[3]]
        for i, (xin, w) in enumerate(zip(inputs, ws_full)):
            # scale-free comparison: the chain's magnitudes grow with every product
            single = kernels.fused_matmul(xin, w)
            same(vals[i], single, f"rank {rank}: tagged chain {what}, launch {i}")
        dist.barrier()

    check_chain(run_chain(), "eager")
    check_chain(run_chain(), "eager again")
    st = torch.cuda.Stream(dev)
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            outs = run_chain()
    for rep in range(3):
        with torch.cuda.stream(st):
            g.replay()
        st.synchronize()
        check_chain(outs, f"graph replay {rep}")
    import ctypes
    from gguf_jax_b200 import _lib
    word = ctypes.c_int32(0)
    assert _lib.lib().ggq_read_status(dev.index, ctypes.byref(word)) == 0 and word.value == 0
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK world={world}", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
