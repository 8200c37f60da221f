"""Device plumbing shared by the host-side modules: torch tensors, streams, scratch.

PyTorch is used for device memory, streams and process groups only; every computation on
quantized data goes through the C ABI in include/ggq.h.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib

_DTYPE_CODE = {torch.float32: _lib.GGQ_F32, torch.bfloat16: _lib.GGQ_BF16, torch.float16: _lib.GGQ_F16}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_stagings: dict[tuple[int, int], torch.Tensor] = {}


def canon_dtype(dtype) -> torch.dtype:
    """Accept torch dtypes, numpy dtypes and names ('bfloat16', 'float32', ...)."""
    if isinstance(dtype, torch.dtype):
        return dtype
    name = getattr(dtype, "name", None) or getattr(dtype, "__name__", None) or str(dtype)
    name = str(name).replace("torch.", "")
    try:
        return getattr(torch, np.dtype(name).name)
    except TypeError:
        pass
    out = getattr(torch, name, None)
    if not isinstance(out, torch.dtype):
        raise TypeError(f"unsupported dtype {dtype!r}")
    return out


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"the kernels write float32, bfloat16 or float16, not {dtype}") from None


def default_device() -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def as_tensor(data, device=None) -> torch.Tensor:
    """numpy / torch / buffer -> torch tensor on ``device`` (default: the current CUDA
    device when there is one), mirroring ``jnp.asarray`` in the reference."""
    if isinstance(data, torch.Tensor):
        return data if device is None else data.to(device)
    t = torch.as_tensor(np.ascontiguousarray(data))
    return t.to(default_device() if device is None else device)


def require_cuda(t: torch.Tensor, what: str) -> int:
    if not t.is_cuda:
        raise RuntimeError(
            f"{what}: the data lives on {t.device}; this library computes on a CUDA device only "
            "(there is no CPU fallback). Move the array to a B200 first.")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def stream_ptr(device_index: int) -> int:
    return torch.cuda.current_stream(device_index).cuda_stream


def staging(device_index: int, nbytes: int, stream: int | None = None) -> torch.Tensor:
    """Device buffer that receives host-resident activations, one per (device, stream), grown on demand.
    Calls on one stream are ordered, so one buffer serves them all.  ``stream``: the current stream's handle if
    the caller already has it."""
    key = (device_index, stream_ptr(device_index) if stream is None else stream)
    buf = _stagings.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _stagings[key] = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=torch.device("cuda", device_index))
    return buf


def workspace(device_index: int, nbytes: int, stream: int | None = None) -> torch.Tensor | None:
    """Zero-filled scratch for the fused kernels, one per (device, stream), grown on demand.
    The kernels leave it zeroed, so it is cleared only when (re)allocated.  ``stream``: the current stream's
    handle if the caller already has it."""
    if nbytes == 0:
        return None
    key = (device_index, stream_ptr(device_index) if stream is None else stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", device_index))
        _workspaces[key] = ws
    return ws
