"""Helpers shared by the op wrappers: stream handles, pointers, scratch buffers."""
from __future__ import annotations

import threading

import torch

from .. import _native

_SCRATCH: dict[tuple, torch.Tensor] = {}


_TLS = threading.local()


def stream_ptr() -> int:
    """The current stream's handle. Also binds the current device's context to this thread the first time
    the thread comes through here: PyTorch's backward threads may not have a driver context yet."""
    dev = torch.cuda.current_device()
    if getattr(_TLS, "device", None) != dev:
        _native.check(_native.lib().idrak_bind_device(dev), "idrak_bind_device")
        _TLS.device = dev
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def scratch(name: str, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A grow-only scratch buffer per (name, dtype, device, stream). Contents are undefined on return.

    Buffers are keyed by the current stream so two streams never share one. While a CUDA graph is being
    captured a fresh tensor comes from the graph's private pool instead (a cached buffer allocated
    outside the capture could be reused by eager work between replays).
    """
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(max(numel, 1), dtype=dtype, device=device)
    key = (name, dtype, device.index, torch.cuda.current_stream().cuda_stream)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1), dtype=dtype, device=device)
        _SCRATCH[key] = buf
    return buf


def release_scratch() -> None:
    _SCRATCH.clear()


def require_cuda_lib() -> None:
    if not _native.available():
        raise RuntimeError("idrak_b200 native library is not built; run `python -m idrak_b200.build`")


def is_bf16_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16
