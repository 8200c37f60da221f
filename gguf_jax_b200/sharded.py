"""Output-row sharding of a quantized weight across the GPUs of one node.

The reference has no multi-device code; this module adds the one strategy the path admits:
``w`` is ``(N, K)`` with rows = output features stored row-major, so a row range is a
contiguous byte slice that never cuts a block.  Every rank keeps ``N / P`` rows, multiplies
the replicated activation with the same fused kernels, and one all-gather along the output
axis rebuilds the replicated ``y`` (NCCL over NVLink when the process group is ``nccl``).

One process per GPU; process-group plumbing is ``torch.distributed``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _backend, _lib, _matmul
from .array import QuantizedArray

__all__ = ["row_range", "shard_rows", "sharded_matmul", "gather_columns", "PeerOutput", "TaggedExchange",
           "TaggedVector"]


def row_range(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows ``[lo, hi)`` of rank ``rank``: equal blocks; ``n_rows`` must divide evenly so that
    the all-gather is uniform (true for every decoder-layer shape; pad the weight otherwise)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    if n_rows % world:
        raise ValueError(f"{n_rows} output rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def shard_rows(w: QuantizedArray, rank: int, world: int, device=None) -> QuantizedArray:
    """This rank's row slice of a 2-D quantized weight, as its own QuantizedArray."""
    if len(w.shape) != 2:
        raise ValueError(f"w must be 2D, got shape {w.shape}")
    lo, hi = row_range(w.shape[0], rank, world)
    data = w.data[lo:hi]
    data = data.to(device) if device is not None else data
    return QuantizedArray(data=data.contiguous(), qtype=w.qtype, shape=(hi - lo, w.shape[1]), dtype=w.dtype)


def gather_columns(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather ``y_local (..., N/P)`` along the last axis into ``(..., N)``.

    The collective moves ``[P, M, N/P]``; the result is returned in the caller's layout.  For a
    single batch row (decode) the gathered buffer already *is* the row, so nothing is permuted.
    """
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    lead = y_local.shape[:-1]
    per = y_local.shape[-1]
    flat = y_local.reshape(-1, per).contiguous()
    m = flat.shape[0]
    if out is None:
        out = torch.empty((world, m, per), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out.view(-1), flat.view(-1), group=group)
    if m == 1:
        return out.reshape(*lead, world * per)
    return out.permute(1, 0, 2).reshape(*lead, world * per)


def sharded_matmul(x: torch.Tensor, w_shard: QuantizedArray, group=None, **kw) -> torch.Tensor:
    """``x @ w.T`` for a row-sharded ``w``: local fused multiply, then the all-gather."""
    return gather_columns(_matmul.matmul(x, w_shard, **kw), group)


class PeerOutput:
    """Replicated output buffers that the fused kernels fill on every rank at once.

    Instead of ``y_local`` followed by an all-gather, :meth:`matmul` launches the kernel behind
    ``ggq_gemv_sharded``: it stores this rank's slice of the output rows straight into every
    rank's copy of ``y`` through peer-mapped pointers (NVLink), and raises a per-rank flag on all
    ranks when its grid has finished.  A following :meth:`matmul` (with ``wait_previous=True``)
    begins by waiting for everybody's flag, so a chain of sharded layers needs no collective
    call and no host synchronisation between layers.

    The buffers live in symmetric memory (``torch.distributed._symmetric_memory``), which provides
    the peer mappings; two output buffers alternate so that a rank that runs ahead never
    overwrites activations a slower rank is still reading.
    """

    def __init__(self, group, max_batch: int, n_total: int, dtype=torch.bfloat16, device=None, n_buffers: int = 2):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        self.device = torch.device(device) if device is not None else _backend.default_device()
        self.dtype = _backend.canon_dtype(dtype)
        self.n_total = int(n_total)
        self.max_batch = int(max_batch)
        self._bufs, self._buf_ptrs = [], []
        for _ in range(n_buffers):
            t = symm.empty((self.max_batch, self.n_total), dtype=self.dtype, device=self.device)
            hdl = symm.rendezvous(t, self.group)
            self._bufs.append(t)
            self._buf_ptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs]))
        flags = symm.empty((64,), dtype=torch.int32, device=self.device)
        flags.zero_()
        hdl = symm.rendezvous(flags, self.group)
        self._flags = flags
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        self._turn = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def matmul(self, x: torch.Tensor, w_shard: QuantizedArray, wait_previous: bool = True) -> torch.Tensor:
        """Launch the fused multiply + exchange; returns this rank's ``(M, n_total)`` buffer.  Its
        contents are complete once every rank's launch has finished (the next fused launch waits for
        that on the device; host code must synchronise and pass a barrier before reading it)."""
        if len(w_shard.shape) != 2 or x.shape[-1] != w_shard.shape[1]:
            raise ValueError(f"contraction mismatch: x {tuple(x.shape)}, w {w_shard.shape}")
        n_out = w_shard.shape[0] * self.world
        if n_out > self.n_total:
            raise ValueError(f"{self.world} shards of {w_shard.shape[0]} rows exceed the buffers' {self.n_total} columns")
        k = w_shard.shape[1]
        # a 2-D view with unit inner stride is passed as it is (row stride = ldx): slicing the leading columns of an
        # earlier exchange's buffer must not launch a copy, which would read the buffer before the peers' stores have landed
        if x.dim() == 2 and x.stride(1) == 1 and x.shape[0] > 1 and x.stride(0) >= k and (x.stride(0) * 2) % 16 == 0 \
                and x.data_ptr() % 16 == 0:
            xm, ldx = x, x.stride(0)
        else:
            xm = x.reshape(-1, k).contiguous()
            ldx = k
        m = xm.shape[0]
        if m > self.max_batch:
            raise ValueError(f"batch {m} exceeds the buffers' {self.max_batch}")
        dev = _backend.require_cuda(w_shard.data, "sharded matmul")
        _lib.ensure_tables(dev)
        L = _lib.lib()
        turn = self._turn
        self._turn = (turn + 1) % len(self._bufs)
        with torch.cuda.device(dev):
            ws = _backend.workspace(dev, L.ggq_workspace_bytes(int(w_shard.qtype), w_shard.shape[0], k, m))
            _lib.check(L.ggq_gemm_sharded(
                int(w_shard.qtype), w_shard.data.data_ptr(), w_shard.shape[0], k, xm.data_ptr(), ldx, m,
                self._buf_ptrs[turn], self._flag_ptrs, self.world, self.rank, n_out,
                _backend.dtype_code(self.dtype), 1 if wait_previous else 0,
                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                _backend.stream_ptr(dev)))
        # a narrower product uses the front of the buffer as a dense (m, n_out) array
        return self._bufs[turn].view(-1)[: m * n_out].view(m, n_out)


class TaggedVector:
    """Handle to the result of one :meth:`TaggedExchange.matmul`: ``n`` tagged words in buffer
    ``index`` of the exchange, produced by its ``serial``-th launch."""

    __slots__ = ("owner", "index", "n", "serial")

    def __init__(self, owner, index: int, n: int, serial: int):
        self.owner, self.index, self.n, self.serial = owner, index, n, serial

    def to_tensor(self) -> torch.Tensor:
        """The bf16 values, once every rank's launch has finished (synchronise the stream and pass
        a barrier first: the host has no other way to know the words have all landed)."""
        words = self.owner._bufs[self.index][: self.n]
        return words.view(torch.int16).view(-1, 2)[:, 0].contiguous().view(torch.bfloat16).reshape(1, self.n)


class TaggedExchange:
    """Chains of row-sharded batch-1 products whose outputs feed later products, with the exchange
    inside the kernels and no flags or fences (``ggq_gemv_sharded_tagged``).

    Each launch stores its rows into every rank's buffer as self-validating 32-bit words (bf16
    value + 16-bit tag of the exchange); a later launch that takes a :class:`TaggedVector` as its
    activation polls the words it needs until they carry the expected tag.  Buffers are used
    round-robin.  A CTA polls only the chunks of the activation vector that its share of the weight
    touches, so it may store its outputs before another rank's part of that vector has landed; what
    bounds how far one rank runs ahead of another is that a launch starts only after the previous
    launch of its own rank has finished, i.e. has seen the whole of *its* activations.  With results
    consumed at most ``max_back`` launches later, a rank storing exchange e can therefore meet a peer
    still reading exchange ``e - 2 * max_back``: two uses of a buffer must lie at least
    ``2 * max_back + 1`` launches apart (``n_buffers >= 2 * max_back + 1``).  All
    ranks must issue the same sequence of launches.  Tags are derived on the device from a
    per-rank launch counter, so a captured CUDA graph of a whole chain can be replayed.
    Supported: Q4_K, Q5_K and Q6_K weights at batch 1 (the tuned kernels' shapes).

    Replaying a captured chain of L launches repeats its buffer sequence, so the round-robin must
    stay intact across the seam: pick ``n_buffers`` with ``L % n_buffers == 0`` or
    ``L % n_buffers >= 2 * max_back + 1`` (:meth:`buffers_for` does).
    """

    @staticmethod
    def buffers_for(chain_length: int, max_back: int = 2) -> int:
        """Smallest buffer count (at least 3) that keeps every reuse ``2 * max_back + 1`` launches apart
        when a chain of ``chain_length`` launches is replayed back to back."""
        apart = max(3, 2 * max_back + 1)
        for nb in range(apart, 33):
            if chain_length % nb == 0 or chain_length % nb >= apart:
                return nb
        return apart

    def __init__(self, group, n_max: int, device=None, n_buffers: int = 4):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        if n_buffers < 3:
            raise ValueError("at least 3 buffers")
        self.device = torch.device(device) if device is not None else _backend.default_device()
        self.n_max = int(n_max)
        self._bufs, self._buf_ptrs = [], []
        for _ in range(n_buffers):
            t = symm.empty((self.n_max,), dtype=torch.int32, device=self.device)
            t.zero_()
            hdl = symm.rendezvous(t, self.group)
            self._bufs.append(t)
            self._buf_ptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs]))
        self._state = torch.zeros(64, dtype=torch.int32, device=self.device)
        self._serial = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def matmul(self, x, w_shard: QuantizedArray, after: TaggedVector | None = None) -> TaggedVector:
        """``x @ w.T`` for this rank's rows of ``w``; ``x`` is a bf16 tensor of ``K`` elements or the
        :class:`TaggedVector` of an earlier launch (its first ``K`` words are used).  ``after``
        names an earlier result that must have landed completely on this rank before the kernel
        reads its activations (what the flag protocol's ``wait_previous`` gives)."""
        k = w_shard.shape[1]
        n_out = w_shard.shape[0] * self.world
        if n_out > self.n_max:
            raise ValueError(f"{self.world} shards of {w_shard.shape[0]} rows exceed the buffers' {self.n_max} words")
        dev = _backend.require_cuda(w_shard.data, "sharded matmul")
        _lib.ensure_tables(dev)
        L = _lib.lib()
        x_plain = x_tagged = None
        back = 0
        if isinstance(x, TaggedVector):
            if x.owner is not self or x.n < k:
                raise ValueError("x must be a result of this exchange with at least K elements")
            back = self._serial - x.serial + 1
            if back < 1 or back > len(self._bufs) - 2:
                raise ValueError(f"that result is {back} launches old; its buffer may have been reused "
                                 f"(at most {len(self._bufs) - 2} with {len(self._bufs)} buffers)")
            x_tagged = self._bufs[x.index].data_ptr()
        else:
            if x.numel() != k or x.dtype != torch.bfloat16:
                raise ValueError(f"x must be {k} bfloat16 values, got {tuple(x.shape)} {x.dtype}")
            x = x.contiguous()
            x_plain = x.data_ptr()
        after_ptr, after_words, after_back = None, 0, 0
        if after is not None:
            after_back = self._serial - after.serial + 1
            if after.owner is not self or after_back < 1 or after_back > len(self._bufs) - 2:
                raise ValueError("`after` must be a recent result of this exchange")
            after_ptr, after_words = self._bufs[after.index].data_ptr(), after.n // 4 * 4
        self._serial += 1
        index = self._serial % len(self._bufs)
        with torch.cuda.device(dev):
            ws = _backend.workspace(dev, L.ggq_workspace_bytes(int(w_shard.qtype), w_shard.shape[0], k, 1))
            _lib.check(L.ggq_gemv_sharded_tagged(
                int(w_shard.qtype), w_shard.data.data_ptr(), w_shard.shape[0], k, x_plain, x_tagged, back,
                after_ptr, after_words, after_back, self._buf_ptrs[index], self._state.data_ptr(), self.world, self.rank, n_out,
                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                _backend.stream_ptr(dev)))
        return TaggedVector(self, index, n_out, self._serial)
