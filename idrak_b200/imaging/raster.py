"""Exact area-coverage rasterisation of outlines (glyphs, shapes) into 8-bit or float coverage masks.

An outline is a list of closed contours made of line, quadratic and cubic segments. Curves are flattened on the host
to line segments within a tolerance; every segment then adds signed trapezoid areas to an accumulation buffer, and a
prefix sum along each row turns the buffer into per-pixel covered area (non-zero or even-odd rule). The result is
the analytic area of the polygon inside each pixel (for non-overlapping contours), not a supersampled estimate.

CPU tensors use a NumPy restatement of the same math (`coverage_reference`); CUDA tensors run
``csrc/raster.cu: coverage_accumulate / coverage_resolve`` - many glyphs rasterise in one launch through the
per-segment image index.

    path = Path().move_to(2, 2).line_to(30, 4).quad_to(40, 20, 20, 30).close()
    mask = rasterize([path], width=48, height=40, device="cuda")     # uint8 [1, 40, 48]

Reference: the reference's ``CoverageRasterizer`` (src/Idrak.Imaging/Fonts: exact coverage of TrueType / CFF outlines on
the CPU), which its page synthesiser draws text with.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..ops._util import stream_ptr


class Path:
    """Contours as drawing commands in pixel units (y down). ``transform`` maps font units to pixels."""

    def __init__(self):
        self.contours: List[List[tuple]] = []      # per contour: [("M", x, y), ("L", x, y), ("Q", cx, cy, x, y), ("C", ...)]

    def move_to(self, x: float, y: float) -> "Path":
        self.contours.append([("M", float(x), float(y))])
        return self

    def line_to(self, x: float, y: float) -> "Path":
        self.contours[-1].append(("L", float(x), float(y)))
        return self

    def quad_to(self, cx: float, cy: float, x: float, y: float) -> "Path":
        self.contours[-1].append(("Q", float(cx), float(cy), float(x), float(y)))
        return self

    def cubic_to(self, c1x: float, c1y: float, c2x: float, c2y: float, x: float, y: float) -> "Path":
        self.contours[-1].append(("C", float(c1x), float(c1y), float(c2x), float(c2y), float(x), float(y)))
        return self

    def close(self) -> "Path":
        return self                                   # contours are closed when flattened

    def transformed(self, sx: float, sy: float, dx: float = 0.0, dy: float = 0.0, shear: float = 0.0) -> "Path":
        """x' = sx x + shear y + dx,  y' = sy y + dy."""
        out = Path()
        for contour in self.contours:
            new = []
            for cmd in contour:
                pts = cmd[1:]
                new.append((cmd[0],) + tuple(v for i in range(0, len(pts), 2)
                                             for v in (sx * pts[i] + shear * pts[i + 1] + dx, sy * pts[i + 1] + dy)))
            out.contours.append(new)
        return out

    def flatten(self, tolerance: float = 0.02) -> np.ndarray:
        """Line segments ``[n, 4]`` (x0, y0, x1, y1), float32; every contour closed back to its start."""
        segs: List[Tuple[float, float, float, float]] = []
        for contour in self.contours:
            if not contour:
                continue
            sx, sy = contour[0][1], contour[0][2]
            x, y = sx, sy
            for cmd in contour[1:]:
                if cmd[0] == "L":
                    segs.append((x, y, cmd[1], cmd[2]))
                    x, y = cmd[1], cmd[2]
                elif cmd[0] == "Q":
                    cx, cy, ex, ey = cmd[1:]
                    # the deviation of a quadratic from its chord over n equal parameter steps is |p0 - 2c + p1| / (4 n^2)
                    dd = math.hypot(x - 2 * cx + ex, y - 2 * cy + ey)
                    n = max(1, int(math.ceil(math.sqrt(dd / (4 * tolerance)))))
                    px, py = x, y
                    for i in range(1, n + 1):
                        t = i / n
                        a, b, c = (1 - t) * (1 - t), 2 * t * (1 - t), t * t
                        qx, qy = a * x + b * cx + c * ex, a * y + b * cy + c * ey
                        segs.append((px, py, qx, qy))
                        px, py = qx, qy
                    x, y = ex, ey
                elif cmd[0] == "C":
                    c1x, c1y, c2x, c2y, ex, ey = cmd[1:]
                    dd = max(math.hypot(x - 2 * c1x + c2x, y - 2 * c1y + c2y),
                             math.hypot(c1x - 2 * c2x + ex, c1y - 2 * c2y + ey))
                    n = max(1, int(math.ceil(math.sqrt(3 * dd / (4 * tolerance)))))
                    px, py = x, y
                    for i in range(1, n + 1):
                        t = i / n
                        u = 1 - t
                        a, b, c, d = u * u * u, 3 * u * u * t, 3 * u * t * t, t * t * t
                        qx, qy = a * x + b * c1x + c * c2x + d * ex, a * y + b * c1y + c * c2y + d * ey
                        segs.append((px, py, qx, qy))
                        px, py = qx, qy
                    x, y = ex, ey
            if (x, y) != (sx, sy):
                segs.append((x, y, sx, sy))
        return np.asarray(segs, np.float32).reshape(-1, 4)


def rect(x0: float, y0: float, x1: float, y1: float) -> Path:
    return Path().move_to(x0, y0).line_to(x1, y0).line_to(x1, y1).line_to(x0, y1).close()


def ellipse(cx: float, cy: float, rx: float, ry: float) -> Path:
    k = 0.5522847498307936           # cubic approximation of a quarter circle
    p = Path().move_to(cx + rx, cy)
    p.cubic_to(cx + rx, cy + k * ry, cx + k * rx, cy + ry, cx, cy + ry)
    p.cubic_to(cx - k * rx, cy + ry, cx - rx, cy + k * ry, cx - rx, cy)
    p.cubic_to(cx - rx, cy - k * ry, cx - k * rx, cy - ry, cx, cy - ry)
    p.cubic_to(cx + k * rx, cy - ry, cx + rx, cy - k * ry, cx + rx, cy)
    return p


# ---------------------------------------------------------------------------------------------------------------------
def accumulate_reference(segs: np.ndarray, width: int, height: int) -> np.ndarray:
    """The accumulation buffer ``[height, width + 1]`` (float64) for line segments - plain loops, the oracle."""
    acc = np.zeros((height, width + 1), np.float64)

    def piece(row, xa, xb, d):
        xm = 0.5 * (xa + xb)
        if xm < 0:
            row[0] += d
        elif xm < width:
            c = min(int(xm), width - 1)
            m = xm - c
            row[c] += d * (1 - m)
            row[c + 1] += d * m

    for x0, y0, x1, y1 in segs.astype(np.float64):
        if y0 == y1:
            continue
        direction = 1.0
        if y0 > y1:
            x0, y0, x1, y1, direction = x1, y1, x0, y0, -1.0
        if y1 <= 0 or y0 >= height:
            continue
        dxdy = (x1 - x0) / (y1 - y0)
        for r in range(max(int(math.floor(y0)), 0), min(int(math.ceil(y1)) - 1, height - 1) + 1):
            ya, yb = max(y0, r), min(y1, r + 1)
            if yb <= ya:
                continue
            xa, xb = x0 + (ya - y0) * dxdy, x0 + (yb - y0) * dxdy
            d = (yb - ya) * direction
            if xa > xb:
                xa, xb = xb, xa
            span = xb - xa
            if span <= 0:
                piece(acc[r], xa, xb, d)
                continue
            if xa < 0:
                cut = min(xb, 0.0)
                acc[r, 0] += d * (cut - xa) / span
                xa = cut
            if xb > width:
                xb = max(xa, float(width))
            x = xa
            while x < xb:
                nxt = min(math.floor(x) + 1.0, xb)
                piece(acc[r], x, nxt, d * (nxt - x) / span)
                x = nxt
    return acc


def resolve_reference(acc: np.ndarray, width: int, rule: str = "nonzero") -> np.ndarray:
    cov = np.abs(np.cumsum(acc, axis=-1)[..., :width])
    if rule == "evenodd":
        cov = cov - 2 * np.floor(cov / 2)
        cov = np.where(cov > 1, 2 - cov, cov)
    else:
        cov = np.minimum(cov, 1.0)
    return cov


def coverage_reference(paths: Sequence[Path], width: int, height: int, rule: str = "nonzero",
                       tolerance: float = 0.02) -> np.ndarray:
    """Float64 coverage ``[len(paths), height, width]`` in 0..1."""
    return np.stack([resolve_reference(accumulate_reference(p.flatten(tolerance), width, height), width, rule)
                     for p in paths]) if len(paths) else np.zeros((0, height, width))


_BOUND = False


def _bind():
    global _BOUND
    if not _BOUND:
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        _native.bind("idrak_coverage_accumulate", i, [vp, vp, i, vp, i, i, i, vp])
        _native.bind("idrak_coverage_resolve", i, [vp, vp, i, ll, i, i, i, vp])
        _BOUND = True


def rasterize(paths: Sequence[Path], width: int, height: int, rule: str = "nonzero", tolerance: float = 0.02,
              device: Optional[str] = None, dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    """Coverage masks ``[len(paths), height, width]``: uint8 (0..255, round to nearest) or float32 (0..1).
    One image per path; all paths of a call go through one pair of kernel launches on CUDA."""
    if rule not in ("nonzero", "evenodd"):
        raise ValueError("rule must be 'nonzero' or 'evenodd'")
    if dtype not in (torch.uint8, torch.float32):
        raise ValueError("dtype must be uint8 or float32")
    dev = torch.device(device) if device is not None else torch.device("cpu")
    n = len(paths)
    if dev.type != "cuda":
        cov = coverage_reference(paths, width, height, rule, tolerance)
        if dtype == torch.uint8:
            return torch.from_numpy(np.rint(cov.astype(np.float32) * np.float32(255.0)).astype(np.uint8))
        return torch.from_numpy(cov.astype(np.float32))
    _bind()
    seg_list = [p.flatten(tolerance) for p in paths]
    counts = [len(s) for s in seg_list]
    out = torch.empty(n, height, width, dtype=dtype, device=dev)
    if n == 0:
        return out
    segs = np.concatenate(seg_list) if sum(counts) else np.zeros((0, 4), np.float32)
    image = np.repeat(np.arange(n, dtype=np.int32), counts)
    pitch = (width + 1 + 3) // 4 * 4
    acc = torch.zeros(n, height, pitch, dtype=torch.float32, device=dev)
    lib = _native.lib()
    if len(segs):
        segs_d = torch.from_numpy(segs).to(dev)
        image_d = torch.from_numpy(image).to(dev)
        rc = lib.idrak_coverage_accumulate(segs_d.data_ptr(), image_d.data_ptr(), len(segs), acc.data_ptr(), width, height,
                                           pitch, stream_ptr())
        _native.check(rc, "idrak_coverage_accumulate")
    rc = lib.idrak_coverage_resolve(acc.data_ptr(), out.data_ptr(), int(dtype == torch.uint8), n * height, width, pitch,
                                    int(rule == "evenodd"), stream_ptr())
    _native.check(rc, "idrak_coverage_resolve")
    return out


def supersample_reference(path: Path, width: int, height: int, factor: int = 16, rule: str = "nonzero",
                          tolerance: float = 0.02) -> np.ndarray:
    """Brute-force coverage by point sampling on a ``factor`` x ``factor`` grid per pixel (winding number per sample);
    slow, independent of the area formulas - a second oracle for tests."""
    segs = path.flatten(tolerance).astype(np.float64)
    ys = (np.arange(height * factor) + 0.5) / factor
    xs = (np.arange(width * factor) + 0.5) / factor
    wind = np.zeros((len(ys), len(xs)), np.int32)
    for x0, y0, x1, y1 in segs:
        if y0 == y1:
            continue
        lo, hi, sign = (y0, y1, 1) if y0 < y1 else (y1, y0, -1)
        rows = np.nonzero((ys >= lo) & (ys < hi))[0]
        if len(rows) == 0:
            continue
        xc = x0 + (ys[rows] - y0) * (x1 - x0) / (y1 - y0)
        # a crossing at xc adds its sign to every sample to its right
        wind[rows[:, None], np.arange(len(xs))[None]] += sign * (xs[None] > xc[:, None])
    inside = (wind % 2 != 0) if rule == "evenodd" else (wind != 0)
    return inside.reshape(height, factor, width, factor).mean(axis=(1, 3))
