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

from . import _matmul
from .array import QuantizedArray

__all__ = ["row_range", "shard_rows", "sharded_matmul", "gather_columns"]


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
