"""Row sharding + all-gather, checked with two CPU ranks over gloo.

The kernels themselves need a GPU, so each rank's local product comes from the CPU oracle here;
what is under test is the host logic that ships: which rows a rank owns, that a shard is a
contiguous byte slice, and that the gathered result has the single-device layout."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from gguf.constants import GGMLQuantizationType as QT

from gguf_jax_b200 import sharded, synth
from oracle import oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, qtype_value, m, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qt = QT(qtype_value)
        n, k = 64, 512
        w = synth.make_weight(n, k, qt, seed=7, device="cpu")
        x = synth.make_x(m, k, seed=8)
        shard = sharded.shard_rows(w, rank, world)
        lo, hi = sharded.row_range(n, rank, world)
        assert shard.shape == (hi - lo, k) and shard.data.is_contiguous()
        assert torch.equal(shard.data, w.data[lo:hi])
        y_local = torch.from_numpy(O.c_matmul(O.bf16_bits(x), shard.data.numpy(), qt)).to(torch.bfloat16)
        y = sharded.gather_columns(y_local)
        full = torch.from_numpy(O.c_matmul(O.bf16_bits(x), w.data.numpy(), qt)).to(torch.bfloat16)
        q.put((rank, bool(torch.equal(y, full)), tuple(y.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [1, 3])
@pytest.mark.parametrize("qtype", [QT.Q4_K, QT.Q6_K], ids=lambda t: t.name)
def test_two_rank_row_sharding_matches_single_device(qtype, m):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, int(qtype), m, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, shape in results:
        assert same, f"rank {rank}: gathered result differs from the single-device product"
        assert shape == (m, 64)


def test_row_range_errors():
    assert sharded.row_range(8192, 3, 8) == (3072, 4096)
    with pytest.raises(ValueError):
        sharded.row_range(10, 0, 4)
    with pytest.raises(ValueError):
        sharded.row_range(8, 4, 4)


def test_tagged_exchange_buffer_count_keeps_reuse_distance_across_replays():
    """A replayed chain of L launches cycles through n buffers; a launch must not land on a buffer that
    one of the 2 * max_back launches before it wrote, across the seam of two replays as well (a rank may
    store exchange e while a peer still reads exchange e - 2 * max_back)."""
    from gguf_jax_b200.sharded import TaggedExchange
    for length in [1, 2, 5, 6, 7, 12, 401, 402, 403, 404, 1000]:
        for max_back in (1, 2, 3):
            nb = TaggedExchange.buffers_for(length, max_back)
            apart = 2 * max_back + 1
            assert nb >= apart
            seq = [(s % nb) for s in range(1, length + 1)] * 3      # three replays, host serials restart
            for i, b in enumerate(seq):
                earlier = seq[max(0, i - (apart - 1)):i]
                if length >= apart:
                    assert b not in earlier, (length, max_back, nb, i)
