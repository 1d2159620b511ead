"""Image-side ops: fused resize + normalise of decoded uint8 images, interpolation and adaptive pooling.

On CUDA tensors the sm_100a kernels of ``csrc/image_ops.cu`` run (forward and backward); on CPU tensors the same
functions call ``torch.nn.functional``, which is also the oracle of the GPU tests.

Reference: Tensor.ResizeNormalize / Interpolate / AdaptiveAvgPool / AdaptiveMaxPool
(src/Idrak.Abstraction/Tensors/Tensor.Resampling.cs) and image preprocessors (src/Idrak.Imaging/Preprocessing).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import _native
from ._util import stream_ptr

_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
    _native.bind("idrak_resize_normalize", i, [vp, vp, i, i, i, i, i, i, i, vp, vp, i, vp])
    _native.bind("idrak_interpolate", i, [vp, vp, i, ll, i, i, i, i, i, i, vp])
    _native.bind("idrak_adaptive_pool", i, [vp, vp, vp, i, ll, i, i, i, i, i, i, vp])
    _BOUND = True


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in (torch.float32, torch.bfloat16)


def resize_normalize(images: torch.Tensor, size: Tuple[int, int], mean: Sequence[float], std: Sequence[float],
                     mode: str = "bilinear", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """uint8 ``[N, H, W, C]`` -> ``dtype`` ``[N, C, OH, OW]``: resize, scale to [0, 1], subtract mean, divide by std."""
    if images.dtype != torch.uint8 or images.dim() != 4:
        raise ValueError("resize_normalize takes uint8 images shaped [N, H, W, C]")
    N, H, W, Cc = images.shape
    OH, OW = size
    if len(mean) != Cc or len(std) != Cc:
        raise ValueError(f"mean / std need {Cc} values")
    if not images.is_cuda:
        x = images.permute(0, 3, 1, 2).float()
        x = F.interpolate(x, size=(OH, OW), mode=mode, **({"align_corners": False} if mode == "bilinear" else {}))
        m = torch.tensor(mean).view(1, Cc, 1, 1)
        s = torch.tensor(std).view(1, Cc, 1, 1)
        return ((x / 255.0 - m) / s).to(dtype)
    _bind()
    out = torch.empty(N, Cc, OH, OW, dtype=dtype, device=images.device)
    m = torch.tensor(list(mean), dtype=torch.float32, device=images.device)
    inv = 1.0 / torch.tensor(list(std), dtype=torch.float32, device=images.device)
    rc = _native.lib().idrak_resize_normalize(images.contiguous().data_ptr(), out.data_ptr(), int(dtype == torch.bfloat16),
                                              N, H, W, Cc, OH, OW, m.data_ptr(), inv.data_ptr(), int(mode == "nearest"),
                                              stream_ptr())
    _native.check(rc, "idrak_resize_normalize")
    return out


class _Interpolate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, OH, OW, bilinear):
        N, Cc, H, W = x.shape
        x = x.contiguous()
        y = torch.empty(N, Cc, OH, OW, dtype=x.dtype, device=x.device)
        rc = _native.lib().idrak_interpolate(x.data_ptr(), y.data_ptr(), int(x.dtype == torch.bfloat16), N * Cc, H, W, OH,
                                             OW, int(bilinear), 0, stream_ptr())
        _native.check(rc, "idrak_interpolate")
        ctx.shape, ctx.bilinear = (N, Cc, H, W, OH, OW), bilinear
        return y

    @staticmethod
    def backward(ctx, dy):
        N, Cc, H, W, OH, OW = ctx.shape
        dy = dy.contiguous()
        dx = torch.empty(N, Cc, H, W, dtype=dy.dtype, device=dy.device)
        rc = _native.lib().idrak_interpolate(dy.data_ptr(), dx.data_ptr(), int(dy.dtype == torch.bfloat16), N * Cc, H, W,
                                             OH, OW, int(ctx.bilinear), 1, stream_ptr())
        _native.check(rc, "idrak_interpolate(backward)")
        return dx, None, None, None


def interpolate(x: torch.Tensor, size: Tuple[int, int], mode: str = "nearest") -> torch.Tensor:
    """``[N, C, H, W]`` -> ``[N, C, OH, OW]``; ``mode``: nearest | bilinear (half-pixel centres)."""
    if mode not in ("nearest", "bilinear"):
        raise ValueError(f"interpolation mode '{mode}' is not supported (nearest, bilinear)")
    if not _native_ok(x):
        return F.interpolate(x, size=tuple(size), mode=mode, **({"align_corners": False} if mode == "bilinear" else {}))
    _bind()
    return _Interpolate.apply(x, int(size[0]), int(size[1]), mode == "bilinear")


class _AdaptivePool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, OH, OW, is_max):
        N, Cc, H, W = x.shape
        x = x.contiguous()
        y = torch.empty(N, Cc, OH, OW, dtype=x.dtype, device=x.device)
        index = torch.empty(N, Cc, OH, OW, dtype=torch.int32, device=x.device) if is_max else None
        rc = _native.lib().idrak_adaptive_pool(x.data_ptr(), y.data_ptr(), index.data_ptr() if is_max else None,
                                               int(x.dtype == torch.bfloat16), N * Cc, H, W, OH, OW, int(is_max), 0,
                                               stream_ptr())
        _native.check(rc, "idrak_adaptive_pool")
        ctx.shape, ctx.is_max = (N, Cc, H, W, OH, OW), is_max
        ctx.save_for_backward(index) if is_max else ctx.save_for_backward()
        return y

    @staticmethod
    def backward(ctx, dy):
        N, Cc, H, W, OH, OW = ctx.shape
        dy = dy.contiguous()
        index = ctx.saved_tensors[0] if ctx.is_max else None
        dx = torch.empty(N, Cc, H, W, dtype=dy.dtype, device=dy.device)
        rc = _native.lib().idrak_adaptive_pool(dy.data_ptr(), dx.data_ptr(), index.data_ptr() if ctx.is_max else None,
                                               int(dy.dtype == torch.bfloat16), N * Cc, H, W, OH, OW, int(ctx.is_max), 1,
                                               stream_ptr())
        _native.check(rc, "idrak_adaptive_pool(backward)")
        return dx, None, None, None


def adaptive_avg_pool(x: torch.Tensor, size: Tuple[int, int]) -> torch.Tensor:
    if not _native_ok(x):
        return F.adaptive_avg_pool2d(x, tuple(size))
    _bind()
    return _AdaptivePool.apply(x, int(size[0]), int(size[1]), False)


def adaptive_max_pool(x: torch.Tensor, size: Tuple[int, int]) -> torch.Tensor:
    if not _native_ok(x):
        return F.adaptive_max_pool2d(x, tuple(size))
    _bind()
    return _AdaptivePool.apply(x, int(size[0]), int(size[1]), True)
