"""Separable image resampling that reproduces Pillow's ``Image.resize`` byte for byte on 8-bit images.

Pillow resizes in two passes (horizontal, then vertical) with per-output-pixel tap tables: for output index ``j`` the
taps cover ``[centre - support, centre + support]`` around ``centre = in0 + (j + 0.5) * scale``, weights come from the
filter kernel evaluated at tap centres, normalised to sum 1. On 8-bit images the weights are rounded to integers with
22 fractional bits and every pass rounds half up and clips to 0..255. This module builds the same tables on the host
and applies them on the CPU (integer tensor ops) or on the GPU (``csrc/raster.cu: resample_pass_*``); float images
use double accumulation and float weights.

    out = resize(images, (out_h, out_w), "bicubic")          # uint8 or float32, [..., H, W, C] or [H, W]

Reference: the reference's ``PillowImageOps`` resampling (src/Idrak.Imaging: box / bilinear / hamming / bicubic /
lanczos with Pillow's arithmetic), which its tests compare with Pillow output byte for byte.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from functools import lru_cache
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..ops._util import stream_ptr

PRECISION_BITS = 32 - 8 - 2


def _box(x: float) -> float:
    return 1.0 if -0.5 < x <= 0.5 else 0.0


def _bilinear(x: float) -> float:
    x = abs(x)
    return 1.0 - x if x < 1.0 else 0.0


def _hamming(x: float) -> float:
    x = abs(x)
    if x == 0.0:
        return 1.0
    if x >= 1.0:
        return 0.0
    x *= math.pi
    return math.sin(x) / x * (0.54 + 0.46 * math.cos(x))


def _bicubic(x: float) -> float:
    a = -0.5
    x = abs(x)
    if x < 1.0:
        return ((a + 2.0) * x - (a + 3.0)) * x * x + 1
    if x < 2.0:
        return (((x - 5) * x + 8) * x - 4) * a
    return 0.0


def _sinc(x: float) -> float:
    if x == 0.0:
        return 1.0
    x *= math.pi
    return math.sin(x) / x


def _lanczos(x: float) -> float:
    return _sinc(x) * _sinc(x / 3) if -3.0 <= x < 3.0 else 0.0


FILTERS = {"box": (_box, 0.5), "bilinear": (_bilinear, 1.0), "hamming": (_hamming, 1.0), "bicubic": (_bicubic, 2.0),
           "lanczos": (_lanczos, 3.0)}


@dataclass(frozen=True)
class Taps:
    """Tap table of one pass: for output ``j`` inputs ``lo[j] .. lo[j] + count[j] - 1`` with weights ``k[j, :count[j]]``."""
    lo: np.ndarray          # int32 [out]
    count: np.ndarray       # int32 [out]
    k: np.ndarray           # float64 [out, ksize]
    ksize: int

    def fixed_point(self) -> np.ndarray:
        """The weights as Pillow stores them for 8-bit images: round half away from zero at 22 fractional bits."""
        scaled = self.k * float(1 << PRECISION_BITS)
        return np.where(scaled < 0, np.trunc(scaled - 0.5), np.trunc(scaled + 0.5)).astype(np.int32)


@lru_cache(maxsize=256)
def taps(in_size: int, out_size: int, filter: str, in0: float = 0.0, in1: Optional[float] = None) -> Taps:
    """Pillow's coefficient table for resizing ``[in0, in1)`` of an axis of ``in_size`` samples to ``out_size``."""
    fn, support0 = FILTERS[filter]
    in1 = float(in_size) if in1 is None else in1
    scale = (in1 - in0) / out_size
    filterscale = max(scale, 1.0)
    support = support0 * filterscale
    ksize = int(math.ceil(support)) * 2 + 1
    lo = np.zeros(out_size, np.int32)
    count = np.zeros(out_size, np.int32)
    k = np.zeros((out_size, ksize), np.float64)
    ss = 1.0 / filterscale
    for j in range(out_size):
        center = in0 + (j + 0.5) * scale
        xmin = max(int(center - support + 0.5), 0)
        xmax = min(int(center + support + 0.5), in_size)
        n = xmax - xmin
        w = np.array([fn((x + xmin - center + 0.5) * ss) for x in range(n)], np.float64)
        total = 0.0
        for v in w:                       # summed left to right, as the C loop does
            total += v
        if total != 0.0:
            w = w / total
        lo[j], count[j] = xmin, n
        k[j, :n] = w
    return Taps(lo, count, k, ksize)


# ---------------------------------------------------------------------------------------------------------------------
_BOUND = False


def _bind():
    global _BOUND
    if not _BOUND:
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        _native.bind("idrak_resample_pass", i, [vp, vp, i, vp, vp, vp, i, ll, i, i, ll, vp])
        _BOUND = True


def _pass_cpu(x: torch.Tensor, t: Taps, axis: int) -> torch.Tensor:
    """Apply one tap table along ``axis`` of a uint8 or float tensor on the CPU."""
    x = x.movedim(axis, -1)
    idx = torch.from_numpy(t.lo.astype(np.int64))[:, None] + torch.arange(t.ksize)[None]
    valid = torch.arange(t.ksize)[None] < torch.from_numpy(t.count.astype(np.int64))[:, None]
    idx = idx.clamp_(max=x.shape[-1] - 1)
    g = x[..., idx]                                           # [..., out, ksize]
    if x.dtype == torch.uint8:
        k = torch.from_numpy(t.fixed_point().astype(np.int64)) * valid
        ss = (g.to(torch.int64) * k).sum(-1) + (1 << (PRECISION_BITS - 1))
        out = (ss >> PRECISION_BITS).clamp_(0, 255).to(torch.uint8)
    else:
        k = torch.from_numpy(t.k) * valid
        out = (g.to(torch.float64) * k).sum(-1).to(x.dtype)
    return out.movedim(-1, axis)


def _pass_cuda(x: torch.Tensor, t: Taps, outer: int, in_len: int, inner: int) -> torch.Tensor:
    _bind()
    dev = x.device
    is_f32 = x.dtype == torch.float32
    k = torch.from_numpy(t.k.astype(np.float32) if is_f32 else t.fixed_point()).to(dev)
    lo, count = torch.from_numpy(t.lo).to(dev), torch.from_numpy(t.count).to(dev)
    out_len = len(t.lo)
    out = torch.empty(outer * out_len * inner, dtype=x.dtype, device=dev)
    rc = _native.lib().idrak_resample_pass(x.data_ptr(), out.data_ptr(), int(is_f32), lo.data_ptr(), count.data_ptr(),
                                           k.data_ptr(), t.ksize, outer, in_len, out_len, inner, stream_ptr())
    _native.check(rc, "idrak_resample_pass")
    return out


def resize(images: torch.Tensor, size: Tuple[int, int], filter: str = "bicubic",
           box: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Resize ``[..., H, W, C]`` (or ``[H, W]``) uint8 / float32 images to ``size = (out_h, out_w)``.

    ``box = (left, top, right, bottom)`` picks the source region (floats allowed), as Pillow's ``box`` argument.
    uint8 results equal ``PIL.Image.resize`` exactly, on the CPU and on the GPU."""
    if filter not in FILTERS:
        raise ValueError(f"unknown filter '{filter}'; known: {', '.join(FILTERS)}")
    if images.dtype not in (torch.uint8, torch.float32):
        raise ValueError("resize takes uint8 or float32 images")
    squeeze = images.dim() == 2
    x = images[..., None] if squeeze else images
    if x.dim() < 3:
        raise ValueError("images must be [..., H, W, C] or [H, W]")
    lead = x.shape[:-3]
    H, W, Cn = x.shape[-3:]
    OH, OW = size
    left, top, right, bottom = box if box is not None else (0.0, 0.0, float(W), float(H))
    if not (0 <= left < right <= W and 0 <= top < bottom <= H):
        raise ValueError("box must lie inside the image")
    need_h = OW != W or left != 0 or right != W
    need_v = OH != H or top != 0 or bottom != H
    x = x.reshape(-1, H, W, Cn).contiguous()
    B = x.shape[0]
    th = taps(W, OW, filter, float(left), float(right)) if need_h else None
    tv = taps(H, OH, filter, float(top), float(bottom)) if need_v else None
    if x.is_cuda:
        if th is not None:
            x = _pass_cuda(x, th, B * H, W, Cn).view(B, H, OW, Cn)
        if tv is not None:
            x = _pass_cuda(x, tv, B, H, x.shape[2] * Cn).view(B, OH, x.shape[2], Cn)
    else:
        if th is not None:
            x = _pass_cpu(x, th, 2)
        if tv is not None:
            x = _pass_cpu(x, tv, 1)
    x = x.reshape(*lead, x.shape[1], x.shape[2], Cn)
    return x[..., 0] if squeeze else x
