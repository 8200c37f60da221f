"""Read a GGUF file into device-resident :class:`QuantizedArray` tensors.

Same public surface as the reference's loader (src/gguf_jax/loader.py:33-73): ``load_gguf(path,
dtype, tensor_filter)`` returns a ``GGUFFile`` with ``metadata`` and ``tensors``.  gguf-py's
``GGUFReader`` memory-maps the file; every tensor's bytes go, still quantized, through one
reusable pinned staging buffer to the device with asynchronous copies.  Two additions for the
multi-GPU case: ``device`` picks the target, and ``shard=(rank, world)`` uploads only this
rank's rows of every 2-D tensor whose row count divides evenly (a row range of the GGUF layout
is a contiguous byte range, so nothing is repacked).
"""
from __future__ import annotations

import dataclasses
from collections.abc import Callable
from typing import Any

import numpy as np
import torch
from gguf.constants import GGMLQuantizationType

from . import _backend
from .array import _NATIVE_TYPES, QuantizedArray

__all__ = ["GGUFFile", "load_gguf"]


@dataclasses.dataclass
class GGUFFile:
    """What a GGUF file holds: key/value metadata and tensors by name."""

    metadata: dict[str, Any]
    tensors: dict[str, QuantizedArray]

    def __repr__(self) -> str:
        return f"GGUFFile({len(self.metadata)} metadata keys, {len(self.tensors)} tensors)"


class _Stager:
    """Host-to-device copies through a pinned buffer that is reused from tensor to tensor (a
    fresh pinned allocation per tensor costs more than the copy for small tensors)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.pinned: torch.Tensor | None = None
        self.busy: torch.cuda.Event | None = None

    def upload(self, host: np.ndarray) -> torch.Tensor:
        src = np.ascontiguousarray(host)
        if self.device.type != "cuda":
            return torch.from_numpy(src.copy())          # the file mapping is read-only: own the bytes
        raw = src.reshape(-1).view(np.uint8)
        if self.busy is not None:
            self.busy.synchronize()      # the previous copy out of the staging buffer has finished
        if self.pinned is None or self.pinned.numel() < raw.size:
            self.pinned = torch.empty(max(raw.size, 1 << 20), dtype=torch.uint8).pin_memory()
        np.copyto(self.pinned.numpy()[: raw.size], raw)
        out = torch.empty(raw.size, dtype=torch.uint8, device=self.device)
        out.copy_(self.pinned[: raw.size], non_blocking=True)
        self.busy = torch.cuda.Event()
        self.busy.record(torch.cuda.current_stream(self.device))
        elem = torch.from_numpy(np.empty(0, dtype=src.dtype)).dtype
        return out.view(elem).reshape(src.shape)


def _metadata(reader) -> dict[str, Any]:
    out = {}
    for key, fld in reader.fields.items():
        try:
            out[key] = fld.contents()
        except Exception:  # noqa: BLE001 -- an unreadable field must not make the tensors unreachable
            out[key] = None
    return out


def load_gguf(path: str, dtype=torch.bfloat16, tensor_filter: Callable[[str], bool] | None = None,
              device=None, shard: tuple[int, int] | None = None) -> GGUFFile:
    """Load ``path``.  Tensors stay in their storage format on ``device`` (default: the current
    CUDA device); ``dtype`` becomes their default decode dtype; ``tensor_filter(name)`` returning
    false skips a tensor.  GGUF lists dimensions innermost first, shapes here are outermost first.
    """
    from gguf import GGUFReader

    target = torch.device(device) if device is not None else _backend.default_device()
    reader = GGUFReader(path, "r")
    stage = _Stager(target)
    tensors: dict[str, QuantizedArray] = {}
    for t in reader.tensors:
        if tensor_filter is not None and not tensor_filter(t.name):
            continue
        qtype = GGMLQuantizationType(t.tensor_type)
        shape = tuple(reversed([int(d) for d in t.shape]))
        host = np.asarray(t.data)
        if qtype not in _NATIVE_TYPES and host.dtype != np.uint8:
            host = np.ascontiguousarray(host).view(np.uint8)     # F32/F16/BF16 arrive as numbers, the kernels take bytes
        if shard is not None and len(shape) == 2 and shape[0] % shard[1] == 0:
            rank, world = shard
            rows = shape[0] // world
            host = host.reshape(shape[0], -1)[rank * rows:(rank + 1) * rows]
            shape = (rows, shape[1])
        tensors[t.name] = QuantizedArray.from_bytes(stage.upload(host), qtype, shape=shape, dtype=dtype)
    if target.type == "cuda":
        torch.cuda.current_stream(target).synchronize()
    return GGUFFile(_metadata(reader), tensors)
