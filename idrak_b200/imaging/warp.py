"""Affine and perspective warps, box blur and rank filters on interleaved images ``[B, H, W, C]`` (uint8 or float32).

The warp follows Pillow's ``Image.transform`` conventions: coefficients map an OUTPUT pixel centre to a source
position, ``u = (a x + b y + c) / (g x + h y + 1)``, ``v = (d x + e y + f) / (g x + h y + 1)``; output pixels whose source
falls outside the image take the fill colour; bilinear and bicubic taps clamp at the border; 8-bit results are
truncated. CUDA tensors run ``csrc/raster.cu``; CPU tensors a NumPy restatement of the same arithmetic.

Reference: the reference's ``PaperTransforms`` (src/Idrak.Imaging/PaperTransforms.cs: rotation, skew, perspective,
page curl built on Pillow-compatible transforms) and the blur / rank filters of ``PillowImageOps``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..ops._util import stream_ptr

TAPS = {"nearest": 0, "bilinear": 1, "bicubic": 2}
_BOUND = False


def _bind():
    global _BOUND
    if not _BOUND:
        vp, i = C.c_void_p, C.c_int
        _native.bind("idrak_warp", i, [vp, vp, i, vp, vp, i, i, i, i, i, i, i, vp])
        _native.bind("idrak_box_blur_u8", i, [vp, vp, i, i, i, i, i, i, vp])
        _native.bind("idrak_rank_filter_u8", i, [vp, vp, i, i, i, i, i, i, vp])
        _BOUND = True


# ---------------------------------------------------------------------------------------------------------------------
# coefficient builders (output -> input, as Pillow wants them)
# ---------------------------------------------------------------------------------------------------------------------
def invert3(m: np.ndarray) -> np.ndarray:
    return np.linalg.inv(np.asarray(m, np.float64).reshape(3, 3))


def coefficients_from_matrix(forward: np.ndarray) -> np.ndarray:
    """8 coefficients from a 3 x 3 matrix that maps INPUT positions to OUTPUT positions."""
    inv = invert3(forward)
    inv = inv / inv[2, 2]
    return inv.reshape(-1)[:8].copy()


def rotation(angle_degrees: float, width: int, height: int, centre: Optional[Tuple[float, float]] = None,
             scale: float = 1.0, translate: Tuple[float, float] = (0.0, 0.0)) -> np.ndarray:
    """Coefficients that rotate the content counter-clockwise about ``centre`` (default: the image centre)."""
    cx, cy = centre if centre is not None else (width / 2.0, height / 2.0)
    t = math.radians(angle_degrees)
    cos, sin = math.cos(t) * scale, math.sin(t) * scale
    fwd = np.array([[cos, sin, cx - cos * cx - sin * cy + translate[0]],
                    [-sin, cos, cy + sin * cx - cos * cy + translate[1]],
                    [0, 0, 1]], np.float64)
    return coefficients_from_matrix(fwd)


def shear(kx: float, ky: float, width: int, height: int) -> np.ndarray:
    cx, cy = width / 2.0, height / 2.0
    fwd = np.array([[1, kx, -kx * cy], [ky, 1, -ky * cx], [0, 0, 1]], np.float64)
    return coefficients_from_matrix(fwd)


def quad_to_quad(src: Sequence[Tuple[float, float]], dst: Sequence[Tuple[float, float]]) -> np.ndarray:
    """Perspective coefficients that send the four ``src`` corners (input image) to the four ``dst`` corners
    (output image)."""
    rows, rhs = [], []
    for (u, v), (x, y) in zip(src, dst):         # solve output (x, y) -> input (u, v)
        rows.append([x, y, 1, 0, 0, 0, -u * x, -u * y]); rhs.append(u)
        rows.append([0, 0, 0, x, y, 1, -v * x, -v * y]); rhs.append(v)
    return np.linalg.solve(np.asarray(rows, np.float64), np.asarray(rhs, np.float64))


# ---------------------------------------------------------------------------------------------------------------------
def _cubic(v1, v2, v3, v4, d):
    p1, p2, p3, p4 = v2, -v1 + v3, 2.0 * (v1 - v2) + v3 - v4, -v1 + v2 - v3 + v4
    return p1 + d * (p2 + d * (p3 + d * p4))


def _warp_cpu(x: np.ndarray, coef: np.ndarray, OH: int, OW: int, taps: int, fill: np.ndarray) -> np.ndarray:
    B, H, W, Cn = x.shape
    out = np.empty((B, OH, OW, Cn), x.dtype)
    ys, xs = np.mgrid[0:OH, 0:OW]
    xs, ys = xs + 0.5, ys + 0.5
    for b in range(B):
        m = coef[b]
        den = m[6] * xs + m[7] * ys + 1.0
        u, v = (m[0] * xs + m[1] * ys + m[2]) / den, (m[3] * xs + m[4] * ys + m[5]) / den
        inside = (u >= 0) & (u < W) & (v >= 0) & (v < H)
        img = x[b].astype(np.float64)
        if taps == 0:
            xi, yi = np.clip(u.astype(np.int64), 0, W - 1), np.clip(v.astype(np.int64), 0, H - 1)
            val = img[yi, xi]
        else:
            uu, vv = u - 0.5, v - 0.5
            x0, y0 = np.floor(uu).astype(np.int64), np.floor(vv).astype(np.int64)
            dx, dy = (uu - x0)[..., None], (vv - y0)[..., None]
            cx = lambda k: np.clip(x0 + k, 0, W - 1)
            if taps == 1:
                ya = np.clip(y0, 0, H - 1)
                r0 = img[ya, cx(0)] + (img[ya, cx(1)] - img[ya, cx(0)]) * dx
                has = ((y0 + 1 >= 0) & (y0 + 1 < H))[..., None]
                yb = np.clip(y0 + 1, 0, H - 1)
                r1 = np.where(has, img[yb, cx(0)] + (img[yb, cx(1)] - img[yb, cx(0)]) * dx, r0)
                val = r0 + (r1 - r0) * dy
            else:
                rows = []
                for t in range(4):
                    yy = np.clip(y0 - 1 + t, 0, H - 1)
                    rows.append(_cubic(img[yy, cx(-1)], img[yy, cx(0)], img[yy, cx(1)], img[yy, cx(2)], dx))
                ok = lambda k: ((y0 + k >= 0) & (y0 + k < H))[..., None]
                rows[0] = np.where(ok(-1), rows[0], rows[1])
                rows[2] = np.where(ok(1), rows[2], rows[1])
                rows[3] = np.where(ok(2), rows[3], rows[2])
                val = _cubic(rows[0], rows[1], rows[2], rows[3], dy)
        if x.dtype == np.uint8 and taps:
            val = np.where(val <= 0, 0, np.where(val >= 255, 255, np.floor(val)))
        out[b] = np.where(inside[..., None], val, fill[None, None]).astype(x.dtype)
    return out


def warp(images: torch.Tensor, coefficients, size: Optional[Tuple[int, int]] = None, mode: str = "bilinear",
         fill: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Warp ``[B, H, W, C]`` (or ``[H, W, C]``) images. ``coefficients``: 8 numbers, or ``[B, 8]`` for one set per image."""
    if mode not in TAPS:
        raise ValueError(f"mode must be one of {', '.join(TAPS)}")
    if images.dtype not in (torch.uint8, torch.float32):
        raise ValueError("warp takes uint8 or float32 images")
    single = images.dim() == 3
    x = images[None] if single else images
    B, H, W, Cn = x.shape
    OH, OW = size if size is not None else (H, W)
    coef = np.asarray(coefficients, np.float64).reshape(-1, 8)
    if coef.shape[0] == 1 and B > 1:
        coef = np.repeat(coef, B, axis=0)
    if coef.shape[0] != B:
        raise ValueError("one coefficient set per image (or one for all)")
    fill_v = np.zeros(Cn, np.float64) if fill is None else np.broadcast_to(np.asarray(fill, np.float64), (Cn,)).copy()
    if not x.is_cuda:
        out = torch.from_numpy(_warp_cpu(x.contiguous().numpy(), coef, OH, OW, TAPS[mode],
                                         fill_v.astype(np.uint8 if x.dtype == torch.uint8 else np.float32)))
    else:
        _bind()
        xc = x.contiguous()
        out = torch.empty(B, OH, OW, Cn, dtype=x.dtype, device=x.device)
        coef_d = torch.from_numpy(np.ascontiguousarray(coef)).to(x.device)
        fill_d = torch.tensor(fill_v, dtype=x.dtype, device=x.device)
        rc = _native.lib().idrak_warp(xc.data_ptr(), out.data_ptr(), int(x.dtype == torch.float32), coef_d.data_ptr(),
                                      fill_d.data_ptr(), B, H, W, Cn, OH, OW, TAPS[mode], stream_ptr())
        _native.check(rc, "idrak_warp")
    return out[0] if single else out


# ---------------------------------------------------------------------------------------------------------------------
def _windows(x: torch.Tensor, ry: int, rx: int) -> torch.Tensor:
    """Edge-replicated windows ``[B, H, W, C, (2 ry + 1)(2 rx + 1)]`` on the CPU."""
    B, H, W, Cn = x.shape
    yi = (torch.arange(H)[:, None] + torch.arange(-ry, ry + 1)[None]).clamp_(0, H - 1)      # [H, ky]
    xi = (torch.arange(W)[:, None] + torch.arange(-rx, rx + 1)[None]).clamp_(0, W - 1)      # [W, kx]
    g = x[:, yi]                      # [B, H, ky, W, C]
    g = g[:, :, :, xi]                # [B, H, ky, W, kx, C]
    return g.permute(0, 1, 3, 5, 2, 4).reshape(B, H, W, Cn, -1)


def box_blur(images: torch.Tensor, radius_x: int, radius_y: Optional[int] = None) -> torch.Tensor:
    """Mean over a ``(2 rx + 1) x (2 ry + 1)`` window with replicated edges, rounded to nearest; uint8 ``[B, H, W, C]``."""
    ry = radius_x if radius_y is None else radius_y
    if images.dtype != torch.uint8 or images.dim() != 4:
        raise ValueError("box_blur takes uint8 images shaped [B, H, W, C]")
    if radius_x == 0 and ry == 0:
        return images.clone()
    if not images.is_cuda:
        w = _windows(images, ry, radius_x).to(torch.int64)
        area = w.shape[-1]
        return ((2 * w.sum(-1) + area) // (2 * area)).to(torch.uint8)
    _bind()
    x = images.contiguous()
    out = torch.empty_like(x)
    B, H, W, Cn = x.shape
    rc = _native.lib().idrak_box_blur_u8(x.data_ptr(), out.data_ptr(), B, H, W, Cn, radius_x, ry, stream_ptr())
    _native.check(rc, "idrak_box_blur_u8")
    return out


def rank_filter(images: torch.Tensor, size: int, rank: int) -> torch.Tensor:
    """The ``rank``-th smallest value (0-based) of each ``size x size`` window, edges replicated. ``rank = 0`` erodes
    bright regions (minimum), ``size * size - 1`` dilates them (maximum), ``size * size // 2`` is the median."""
    if images.dtype != torch.uint8 or images.dim() != 4:
        raise ValueError("rank_filter takes uint8 images shaped [B, H, W, C]")
    if size % 2 == 0 or not 0 <= rank < size * size:
        raise ValueError("size must be odd and 0 <= rank < size * size")
    if not images.is_cuda:
        w = _windows(images, size // 2, size // 2)
        return w.sort(-1).values[..., rank].contiguous()
    _bind()
    x = images.contiguous()
    out = torch.empty_like(x)
    B, H, W, Cn = x.shape
    rc = _native.lib().idrak_rank_filter_u8(x.data_ptr(), out.data_ptr(), B, H, W, Cn, size, rank, stream_ptr())
    _native.check(rc, "idrak_rank_filter_u8")
    return out


def median_filter(images, size=3):
    return rank_filter(images, size, size * size // 2)


def min_filter(images, size=3):
    return rank_filter(images, size, 0)


def max_filter(images, size=3):
    return rank_filter(images, size, size * size - 1)


def gaussian_blur(images: torch.Tensor, sigma: float, passes: int = 3) -> torch.Tensor:
    """A Gaussian approximated by ``passes`` box blurs whose radii give the same variance (a box of radius r has
    variance ((2 r + 1)^2 - 1) / 12)."""
    if sigma <= 0:
        return images.clone()
    ideal = math.sqrt(12.0 * sigma * sigma / passes + 1.0)
    lower = int(ideal) if int(ideal) % 2 == 1 else int(ideal) - 1
    lower = max(lower, 1)
    upper = lower + 2
    n_lower = round((12.0 * sigma * sigma - passes * lower * lower - 4 * passes * lower - 3 * passes) / (-4.0 * lower - 4))
    out = images
    for i in range(passes):
        width = lower if i < n_lower else upper
        out = box_blur(out, (width - 1) // 2)
    return out
