"""Seeded scan / paper effects for synthetic document pages, on uint8 images ``[B, H, W, C]`` (CPU or CUDA).

Every effect is a function ``fn(images, rng, strength) -> images`` registered under a name; ``strength`` in 0..1 scales
how visible it is and ``rng`` (a NumPy generator) draws its parameters, so a pipeline with a fixed seed reproduces
its pages. Per-pixel effects (tone curve, illumination, vignette, noise, fibre) go through one fused pass
(``csrc/raster.cu: paper_effects_kernel`` on CUDA, a NumPy restatement with the same counter-based random numbers on
the CPU); geometric ones use the warps, neighbourhood ones the blur / rank filters, the rest are small tensor
expressions or shapes drawn with the coverage rasteriser.

    page = apply(page, ["rotate_small", "paper_fibre", "gaussian_noise", "defocus"], seed=7)
    page = random_pipeline(page, seed=11, count=5)

Reference: the reference's ``PaperEffects`` / ``PaperTransforms`` (src/Idrak.Imaging/PaperEffects.cs, PaperTransforms.cs:
about fifty seeded effects applied to rendered pages for OCR training data).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import _native
from ..ops._util import stream_ptr
from . import warp as W
from .raster import Path, ellipse, rasterize
from .resample import resize

_BOUND = False
_M64 = (1 << 64) - 1


def _bind():
    global _BOUND
    if not _BOUND:
        vp, i = C.c_void_p, C.c_int
        _native.bind("idrak_paper_effects", i, [vp, vp, i, i, i, i, vp, C.c_ulonglong, vp])
        _BOUND = True


@dataclass
class PixelPass:
    """Parameters of the fused per-pixel pass, applied in this order: tone curve ``gain * v^gamma + bias``, illumination
    gradient, vignette, fibre texture, Gaussian noise, salt and pepper."""
    gain: float = 1.0
    bias: float = 0.0
    gamma: float = 1.0
    grad_x: float = 0.0
    grad_y: float = 0.0
    vignette: float = 0.0
    vignette_power: float = 2.0
    noise_sigma: float = 0.0
    salt: float = 0.0
    pepper: float = 0.0
    fibre: float = 0.0
    fibre_scale: float = 0.25
    grey_noise: bool = True
    seed: int = 0

    def as_floats(self) -> List[float]:
        return [self.gain, self.bias, self.gamma, self.grad_x, self.grad_y, self.vignette, self.vignette_power,
                self.noise_sigma, self.salt, self.pepper, self.fibre, self.fibre_scale, 1.0 if self.grey_noise else 0.0]


# ---------------------------------------------------------------------------------------------------------------------
# the counter-based random numbers of the kernel, restated with NumPy
# ---------------------------------------------------------------------------------------------------------------------
def _mix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _uniform01(seed: int, counter: np.ndarray, stream: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        key = _mix64(np.asarray((seed ^ ((0xD1B54A32D192ED03 * (stream + 1)) & _M64)) & _M64, np.uint64))
        h = _mix64(key + counter.astype(np.uint64))
    return (h >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def _lattice(seed: int, ix: np.ndarray, iy: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        c = (ix.astype(np.int64).astype(np.uint64) & np.uint64(0xFFFFFFFF)) * np.uint64(0x1F123BB5) \
            + (iy.astype(np.int64).astype(np.uint64) & np.uint64(0xFFFFFFFF))
    return _uniform01(seed, c, 7)


def _pixel_pass_cpu(x: np.ndarray, p: PixelPass) -> np.ndarray:
    B, H, Wd, Cn = x.shape
    f32 = np.float32
    v = x.astype(f32) * f32(1.0 / 255.0)
    if p.gamma != 1.0:
        v = np.power(np.maximum(v, 0), f32(p.gamma), dtype=f32)
    v = f32(p.gain) * v + f32(p.bias)
    fx = ((np.arange(Wd, dtype=f32) + f32(0.5)) / f32(Wd) - f32(0.5))[None, None, :, None]
    fy = ((np.arange(H, dtype=f32) + f32(0.5)) / f32(H) - f32(0.5))[None, :, None, None]
    v = v * (f32(1.0) + f32(p.grad_x) * fx + f32(p.grad_y) * fy)
    if p.vignette != 0.0:
        r = np.sqrt(fx * fx + fy * fy) * f32(1.41421356)
        v = v * (f32(1.0) - f32(p.vignette) * np.power(r, f32(p.vignette_power), dtype=f32))
    if p.fibre != 0.0:
        gx = (np.arange(Wd, dtype=f32) * f32(p.fibre_scale))[None, :]
        gy = (np.arange(H, dtype=f32) * f32(p.fibre_scale))[:, None]
        ix, iy = np.floor(gx).astype(np.int64), np.floor(gy).astype(np.int64)
        tx, ty = gx - ix, gy - iy
        tx, ty = tx * tx * (3 - 2 * tx), ty * ty * (3 - 2 * ty)
        ix, iy = np.broadcast_to(ix, (H, Wd)), np.broadcast_to(iy, (H, Wd))
        for b in range(B):
            s = (p.seed + b) & _M64
            n00, n10 = _lattice(s, ix, iy), _lattice(s, ix + 1, iy)
            n01, n11 = _lattice(s, ix, iy + 1), _lattice(s, ix + 1, iy + 1)
            tex = (n00 + (n10 - n00) * tx) * (1 - ty) + (n01 + (n11 - n01) * tx) * ty - f32(0.5)
            v[b] += f32(p.fibre) * tex[..., None].astype(f32)
    pixel = np.arange(B * H * Wd, dtype=np.uint64).reshape(B, H, Wd, 1)
    counter = pixel if p.grey_noise else pixel * np.uint64(Cn) + np.arange(Cn, dtype=np.uint64)[None, None, None]
    if p.noise_sigma != 0.0:
        u1 = np.maximum(_uniform01(p.seed, counter, 1), f32(5.9604645e-8))
        u2 = _uniform01(p.seed, counter, 2)
        v = v + f32(p.noise_sigma) * np.sqrt(f32(-2.0) * np.log(u1)) * np.cos(f32(6.28318531) * u2)
    if p.salt != 0.0 or p.pepper != 0.0:
        u = _uniform01(p.seed, pixel, 3)
        v = np.where(u < f32(p.pepper), f32(0), np.where(u > f32(1.0) - f32(p.salt), f32(1), v))
    return np.rint(np.clip(v, 0, 1) * f32(255.0)).astype(np.uint8)


def pixel_pass(images: torch.Tensor, p: PixelPass) -> torch.Tensor:
    if images.dtype != torch.uint8 or images.dim() != 4:
        raise ValueError("effects take uint8 images shaped [B, H, W, C]")
    if not images.is_cuda:
        return torch.from_numpy(_pixel_pass_cpu(images.contiguous().numpy(), p))
    _bind()
    x = images.contiguous()
    out = torch.empty_like(x)
    B, H, Wd, Cn = x.shape
    params = (C.c_float * 13)(*p.as_floats())
    rc = _native.lib().idrak_paper_effects(x.data_ptr(), out.data_ptr(), B, H, Wd, Cn, params, p.seed & _M64, stream_ptr())
    _native.check(rc, "idrak_paper_effects")
    return out


# ---------------------------------------------------------------------------------------------------------------------
# the registry
# ---------------------------------------------------------------------------------------------------------------------
Effect = Callable[[torch.Tensor, np.random.Generator, float], torch.Tensor]
EFFECTS: Dict[str, Effect] = {}


def effect(name: str):
    def add(fn: Effect) -> Effect:
        EFFECTS[name] = fn
        return fn
    return add


def _seed(rng: np.random.Generator) -> int:
    return int(rng.integers(0, 1 << 62))


def _scale_u8(x: torch.Tensor, gain: torch.Tensor) -> torch.Tensor:
    """x * gain (broadcast), rounded and clipped."""
    return (x.float() * gain).round_().clamp_(0, 255).to(torch.uint8)


def _white(x: torch.Tensor) -> List[float]:
    return [255.0] * x.shape[-1]


@effect("brightness")
def _brightness(x, rng, s):
    return pixel_pass(x, PixelPass(bias=float(rng.uniform(-0.25, 0.25)) * s))


@effect("contrast")
def _contrast(x, rng, s):
    g = 1.0 + float(rng.uniform(-0.5, 0.5)) * s
    return pixel_pass(x, PixelPass(gain=g, bias=0.5 * (1 - g)))


@effect("gamma")
def _gamma(x, rng, s):
    return pixel_pass(x, PixelPass(gamma=float(2.0 ** (rng.uniform(-1, 1) * s))))


@effect("illumination_gradient")
def _illumination(x, rng, s):
    return pixel_pass(x, PixelPass(grad_x=float(rng.uniform(-0.6, 0.6)) * s, grad_y=float(rng.uniform(-0.6, 0.6)) * s))


@effect("vignette")
def _vignette(x, rng, s):
    return pixel_pass(x, PixelPass(vignette=0.6 * s, vignette_power=float(rng.uniform(1.5, 3.0))))


@effect("gaussian_noise")
def _gaussian_noise(x, rng, s):
    return pixel_pass(x, PixelPass(noise_sigma=0.12 * s, seed=_seed(rng)))


@effect("colour_noise")
def _colour_noise(x, rng, s):
    return pixel_pass(x, PixelPass(noise_sigma=0.08 * s, grey_noise=False, seed=_seed(rng)))


@effect("salt_pepper")
def _salt_pepper(x, rng, s):
    return pixel_pass(x, PixelPass(salt=0.01 * s, pepper=0.01 * s, seed=_seed(rng)))


@effect("paper_fibre")
def _paper_fibre(x, rng, s):
    return pixel_pass(x, PixelPass(fibre=0.15 * s, fibre_scale=float(rng.uniform(0.08, 0.5)), seed=_seed(rng)))


@effect("coarse_grain")
def _coarse_grain(x, rng, s):
    return pixel_pass(x, PixelPass(fibre=0.25 * s, fibre_scale=float(rng.uniform(0.01, 0.05)), seed=_seed(rng)))


@effect("faded_ink")
def _faded_ink(x, rng, s):
    return pixel_pass(x, PixelPass(gain=1.0 - 0.5 * s, bias=0.5 * s))


@effect("defocus")
def _defocus(x, rng, s):
    return W.gaussian_blur(x, 0.5 + 2.5 * s * float(rng.uniform(0.3, 1.0)))


@effect("motion_blur_horizontal")
def _motion_h(x, rng, s):
    return W.box_blur(x, max(1, int(round(6 * s * rng.uniform(0.3, 1.0)))), 0)


@effect("motion_blur_vertical")
def _motion_v(x, rng, s):
    return W.box_blur(x, 0, max(1, int(round(6 * s * rng.uniform(0.3, 1.0)))))


@effect("ink_thicken")
def _ink_thicken(x, rng, s):
    return W.min_filter(x, 3 if s < 0.7 else 5)


@effect("ink_thin")
def _ink_thin(x, rng, s):
    return W.max_filter(x, 3)


@effect("median_smooth")
def _median(x, rng, s):
    return W.median_filter(x, 3 if s < 0.7 else 5)


@effect("low_resolution")
def _low_resolution(x, rng, s):
    B, H, Wd, Cn = x.shape
    f = 1.0 / (1.0 + 3.0 * s * float(rng.uniform(0.3, 1.0)))
    small = resize(x, (max(int(H * f), 1), max(int(Wd * f), 1)), "box")
    return resize(small, (H, Wd), "bilinear")


@effect("rotate_small")
def _rotate_small(x, rng, s):
    B, H, Wd, _ = x.shape
    return W.warp(x, W.rotation(float(rng.uniform(-4, 4)) * s, Wd, H), mode="bilinear", fill=_white(x))


@effect("skew")
def _skew(x, rng, s):
    B, H, Wd, _ = x.shape
    return W.warp(x, W.shear(float(rng.uniform(-0.08, 0.08)) * s, float(rng.uniform(-0.03, 0.03)) * s, Wd, H),
                  mode="bilinear", fill=_white(x))


@effect("perspective_tilt")
def _perspective(x, rng, s):
    B, H, Wd, _ = x.shape
    j = lambda: float(rng.uniform(0, 0.06)) * s
    src = [(0, 0), (Wd, 0), (Wd, H), (0, H)]
    dst = [(j() * Wd, j() * H), (Wd - j() * Wd, j() * H), (Wd - j() * Wd, H - j() * H), (j() * Wd, H - j() * H)]
    return W.warp(x, W.quad_to_quad(src, dst), mode="bilinear", fill=_white(x))


@effect("zoom")
def _zoom(x, rng, s):
    B, H, Wd, _ = x.shape
    return W.warp(x, W.rotation(0.0, Wd, H, scale=1.0 + float(rng.uniform(-0.1, 0.1)) * s), mode="bilinear", fill=_white(x))


@effect("translate")
def _translate(x, rng, s):
    B, H, Wd, _ = x.shape
    t = (float(rng.uniform(-0.05, 0.05)) * Wd * s, float(rng.uniform(-0.05, 0.05)) * H * s)
    return W.warp(x, W.rotation(0.0, Wd, H, translate=t), mode="bilinear", fill=_white(x))


@effect("scanner_streaks")
def _streaks(x, rng, s):
    Wd = x.shape[2]
    gain = 1.0 + (rng.random(Wd) < 0.02) * rng.uniform(-0.5, 0.2, Wd) * s
    return _scale_u8(x, torch.tensor(gain, dtype=torch.float32, device=x.device).view(1, 1, Wd, 1))


@effect("toner_bands")
def _bands(x, rng, s):
    H = x.shape[1]
    phase, period = float(rng.uniform(0, 2 * math.pi)), float(rng.uniform(H / 8, H / 2))
    fade = 0.5 * s * (0.5 + 0.5 * np.sin(np.arange(H) * 2 * math.pi / period + phase))
    v = x.float()
    g = torch.tensor(fade, dtype=torch.float32, device=x.device).view(1, H, 1, 1)
    return (v + (255.0 - v) * g).round_().clamp_(0, 255).to(torch.uint8)       # ink fades towards white


@effect("colour_cast")
def _cast(x, rng, s):
    Cn = x.shape[-1]
    g = 1.0 + rng.uniform(-0.15, 0.05, Cn) * s
    return _scale_u8(x, torch.tensor(g, dtype=torch.float32, device=x.device).view(1, 1, 1, Cn))


@effect("yellowing")
def _yellowing(x, rng, s):
    Cn = x.shape[-1]
    g = np.ones(Cn)
    if Cn >= 3:
        g[:3] = [1.0 - 0.02 * s, 1.0 - 0.08 * s, 1.0 - 0.3 * s]
    else:
        g[:] = 1.0 - 0.1 * s
    return _scale_u8(x, torch.tensor(g, dtype=torch.float32, device=x.device).view(1, 1, 1, Cn))


def _mask_multiply(x: torch.Tensor, paths: Sequence[Path], darkness: float, blur: float = 0.0) -> torch.Tensor:
    """Darken x under the union of the paths' coverage (same shapes on every image of the batch)."""
    B, H, Wd, Cn = x.shape
    merged = Path()
    for p in paths:
        merged.contours += p.contours
    m = rasterize([merged], Wd, H, device=str(x.device), dtype=torch.uint8)          # [1, H, W]
    if blur > 0:
        m = W.gaussian_blur(m[..., None], blur)[..., 0]
    gain = 1.0 - darkness * (m.float() / 255.0)
    return _scale_u8(x, gain.view(1, H, Wd, 1))


@effect("fold_line")
def _fold(x, rng, s):
    B, H, Wd, _ = x.shape
    if rng.random() < 0.5:
        y = float(rng.uniform(0.2, 0.8)) * H
        tilt = float(rng.uniform(-0.01, 0.01)) * Wd
        p = Path().move_to(0, y).line_to(Wd, y + tilt).line_to(Wd, y + tilt + 1.5).line_to(0, y + 1.5)
    else:
        xx = float(rng.uniform(0.2, 0.8)) * Wd
        tilt = float(rng.uniform(-0.01, 0.01)) * H
        p = Path().move_to(xx, 0).line_to(xx + 1.5, 0).line_to(xx + tilt + 1.5, H).line_to(xx + tilt, H)
    return _mask_multiply(x, [p], 0.5 * s, blur=1.0)


@effect("stains")
def _stains(x, rng, s):
    B, H, Wd, _ = x.shape
    blobs = [ellipse(float(rng.uniform(0, Wd)), float(rng.uniform(0, H)), float(rng.uniform(0.03, 0.15)) * Wd,
                     float(rng.uniform(0.03, 0.15)) * H) for _ in range(int(rng.integers(1, 4)))]
    return _mask_multiply(x, blobs, 0.25 * s, blur=max(Wd, H) / 100.0)


@effect("dust")
def _dust(x, rng, s):
    B, H, Wd, _ = x.shape
    n = max(1, int(40 * s))
    specks = [ellipse(float(rng.uniform(0, Wd)), float(rng.uniform(0, H)), float(rng.uniform(0.4, 1.6)),
                      float(rng.uniform(0.4, 1.6))) for _ in range(n)]
    return _mask_multiply(x, specks, 0.8)


@effect("spine_shadow")
def _spine(x, rng, s):
    B, H, Wd, _ = x.shape
    left = rng.random() < 0.5
    t = torch.linspace(0, 1, Wd, device=x.device)
    d = t if left else 1 - t
    gain = 1.0 - 0.6 * s * torch.exp(-d / float(rng.uniform(0.03, 0.12)))
    return _scale_u8(x, gain.view(1, 1, Wd, 1))


@effect("edge_darkening")
def _edges(x, rng, s):
    B, H, Wd, _ = x.shape
    ty = torch.linspace(0, 1, H, device=x.device).view(H, 1)
    tx = torch.linspace(0, 1, Wd, device=x.device).view(1, Wd)
    d = torch.minimum(torch.minimum(tx, 1 - tx), torch.minimum(ty, 1 - ty))
    gain = 1.0 - 0.5 * s * torch.exp(-d / float(rng.uniform(0.01, 0.05)))
    return _scale_u8(x, gain.view(1, H, Wd, 1))


@effect("binarize")
def _binarize(x, rng, s):
    t = 128 + int(rng.uniform(-60, 60) * s)
    grey = x.float().mean(-1, keepdim=True)
    return torch.where(grey >= t, 255, 0).to(torch.uint8).expand_as(x).contiguous()


@effect("posterize")
def _posterize(x, rng, s):
    bits = max(1, 8 - int(round(5 * s)))
    mask = (0xFF << (8 - bits)) & 0xFF
    return x & mask


@effect("bleed_through")
def _bleed(x, rng, s):
    back = W.gaussian_blur(torch.flip(x, dims=[2]), 1.5)            # the mirrored page showing through
    v, b = x.float(), back.float()
    return (v - (255.0 - b) * (0.25 * s)).round_().clamp_(0, 255).to(torch.uint8)


def _dct8(device) -> torch.Tensor:
    k = torch.arange(8, dtype=torch.float32, device=device)
    m = torch.cos((2 * k[None] + 1) * k[:, None] * math.pi / 16) * math.sqrt(2 / 8)
    m[0] = m[0] / math.sqrt(2)
    return m


@effect("block_compression")
def _blocks(x, rng, s):
    """8 x 8 block transform coding with a coarse quantiser: the blocking and ringing of a heavily compressed scan."""
    B, H, Wd, Cn = x.shape
    Hp, Wp = (H + 7) // 8 * 8, (Wd + 7) // 8 * 8
    v = torch.nn.functional.pad(x.permute(0, 3, 1, 2).float(), (0, Wp - Wd, 0, Hp - H), mode="replicate") - 128.0
    d = _dct8(x.device)
    blocks = v.view(B, Cn, Hp // 8, 8, Wp // 8, 8).permute(0, 1, 2, 4, 3, 5)
    coef = d @ blocks @ d.t()
    i = torch.arange(8, device=x.device, dtype=torch.float32)
    q = (1.0 + (i[:, None] + i[None]) * 1.5) * (2.0 + 30.0 * s)
    coef = torch.round(coef / q) * q
    rec = (d.t() @ coef @ d).permute(0, 1, 2, 4, 3, 5).reshape(B, Cn, Hp, Wp)[:, :, :H, :Wd] + 128.0
    return rec.round_().clamp_(0, 255).to(torch.uint8).permute(0, 2, 3, 1).contiguous()


@effect("invert_region")
def _invert_region(x, rng, s):
    """A highlighted (reverse video) horizontal band, as a marker pen or a redaction leaves."""
    B, H, Wd, _ = x.shape
    y0 = int(rng.uniform(0.1, 0.8) * H)
    y1 = min(H, y0 + max(2, int(0.04 * H)))
    out = x.clone()
    band = out[:, y0:y1].float()
    out[:, y0:y1] = (band * (1.0 - 0.35 * s)).round_().to(torch.uint8)
    return out


# ---------------------------------------------------------------------------------------------------------------------
def apply(images: torch.Tensor, names: Sequence[str], seed: int = 0, strength: float = 0.5) -> torch.Tensor:
    """Run the named effects in order; effect ``i`` draws from a generator seeded by ``(seed, i)``."""
    single = images.dim() == 3
    x = images[None] if single else images
    for i, name in enumerate(names):
        if name not in EFFECTS:
            raise KeyError(f"unknown effect '{name}'; known: {', '.join(sorted(EFFECTS))}")
        x = EFFECTS[name](x, np.random.default_rng([seed, i]), strength)
    return x[0] if single else x


def random_pipeline(images: torch.Tensor, seed: int = 0, count: int = 4, strength: Optional[float] = None,
                    allowed: Optional[Sequence[str]] = None) -> torch.Tensor:
    """Pick ``count`` distinct effects and a strength from the seed and apply them (geometry first, then tone and
    texture, then blur and noise - the order a page meets them on its way through a scanner)."""
    rng = np.random.default_rng([seed, 0x5EED])
    pool = sorted(allowed if allowed is not None else EFFECTS)
    picks = list(rng.choice(pool, size=min(count, len(pool)), replace=False))
    order = {n: i for i, n in enumerate(STAGE_ORDER)}
    picks.sort(key=lambda n: order.get(n, len(order)))
    return apply(images, picks, seed, float(rng.uniform(0.2, 0.9)) if strength is None else strength)


STAGE_ORDER = ["perspective_tilt", "rotate_small", "skew", "zoom", "translate", "ink_thicken", "ink_thin", "faded_ink",
               "bleed_through", "fold_line", "stains", "dust", "paper_fibre", "coarse_grain", "yellowing", "colour_cast",
               "illumination_gradient", "vignette", "spine_shadow", "edge_darkening", "toner_bands", "scanner_streaks",
               "brightness", "contrast", "gamma", "defocus", "motion_blur_horizontal", "motion_blur_vertical",
               "median_smooth", "low_resolution", "gaussian_noise", "colour_noise", "salt_pepper", "invert_region",
               "posterize", "block_compression", "binarize"]
