"""GGUF file -> dict of device-resident QuantizedArrays.

Stands for src/gguf_jax/loader.py:33-73.  Parsing is delegated to gguf-py's GGUFReader
(memory-mapped); each tensor's raw bytes are staged through pinned host memory and
uploaded without dequantizing.
"""
from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
from gguf.constants import GGMLQuantizationType

from . import _backend
from .array import _NATIVE_TYPES, QuantizedArray

__all__ = ["GGUFFile", "load_gguf"]


@dataclass
class GGUFFile:
    """Contents of a GGUF file: metadata key-values and named tensors (a plain dict of
    :class:`QuantizedArray`, so it composes with pytree utilities)."""

    metadata: dict[str, Any]
    tensors: dict[str, QuantizedArray]

    def __repr__(self) -> str:
        return f"GGUFFile({len(self.metadata)} metadata keys, {len(self.tensors)} tensors)"


def _field_value(fld) -> Any:
    try:
        return fld.contents()
    except Exception:  # noqa: BLE001 -- exotic field layouts must not fail the load
        return None


def _upload(host: np.ndarray, device: torch.device) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(host))
    if device.type == "cuda":
        return t.pin_memory().to(device, non_blocking=True)
    return t.clone()


def load_gguf(path: str, dtype=torch.bfloat16, tensor_filter: Callable[[str], bool] | None = None,
              device=None) -> GGUFFile:
    """Load a GGUF file; payloads stay quantized (uint8) on ``device`` (default: the
    current CUDA device).  ``tensor_filter`` skips tensors whose name it rejects."""
    from gguf import GGUFReader

    device = torch.device(device) if device is not None else _backend.default_device()
    reader = GGUFReader(path, "r")
    metadata = {name: _field_value(fld) for name, fld in reader.fields.items()}
    tensors: dict[str, QuantizedArray] = {}
    for entry in reader.tensors:
        if tensor_filter is not None and not tensor_filter(entry.name):
            continue
        qtype = GGMLQuantizationType(entry.tensor_type)
        shape = tuple(int(d) for d in entry.shape.tolist())[::-1]  # GGUF stores dims innermost-first
        raw = entry.data
        if qtype not in _NATIVE_TYPES:
            raw = np.ascontiguousarray(raw).view(np.uint8)  # F16/F32 arrive as native dtypes
        tensors[entry.name] = QuantizedArray.from_bytes(_upload(raw, device), qtype, shape=shape, dtype=dtype)
    if device.type == "cuda":
        torch.cuda.current_stream(device).synchronize()
    return GGUFFile(metadata=metadata, tensors=tensors)
