"""Element-wise operations with their gradients: one unary family, one binary family, fused multiply-add, selection,
fill, row-vector add and mask-free dropout. CUDA fp32 / bf16 tensors run the kernels of ``csrc/pointwise.cu``; anything
else (CPU, other dtypes) runs the plain PyTorch statement beside each function, which is also the test oracle.

Reference: the element-wise part of ``Tensor`` (src/Idrak.Abstraction/Tensors/Tensor.cs, Tensor.Pointwise.cs) and its
device kernels (src/Idrak.Gpu/Cuda/PtxKernels.cs:31-39, PtxKernels.Pointwise.cs, PtxKernels.Advanced.cs:12).
"""
from __future__ import annotations

import math

import torch

from .. import _native
from ._util import ptr, stream_ptr

UNARY = {name: i for i, name in enumerate(
    ["affine", "sigmoid", "tanh", "relu", "square", "abs", "sqrt", "sin", "cos", "silu", "sign", "exp", "log", "gelu",
     "gelu_erf", "inv_sqrt", "pow", "clamp", "leaky_relu", "neg", "reciprocal"])}
BINARY = {name: i for i, name in enumerate(["add", "sub", "mul", "div", "max", "min", "axpby"])}
_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def _native_ok(*ts: torch.Tensor) -> bool:
    t0 = ts[0]
    return (t0.is_cuda and t0.dtype in _DTYPES and t0.numel() > 0
            and all(t.is_cuda and t.dtype == t0.dtype and t.shape == t0.shape for t in ts))


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# ----------------------------------------------------------------------------------------------------------- references
def unary_reference(name: str, x: torch.Tensor, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
    f = x.float()
    out = {
        "affine": lambda: a * f + b, "sigmoid": lambda: torch.sigmoid(f), "tanh": lambda: torch.tanh(f),
        "relu": lambda: torch.relu(f), "square": lambda: f * f, "abs": lambda: f.abs(), "sqrt": lambda: f.sqrt(),
        "sin": lambda: f.sin(), "cos": lambda: f.cos(), "silu": lambda: torch.nn.functional.silu(f),
        "sign": lambda: f.sign(), "exp": lambda: f.exp(), "log": lambda: f.log(),
        "gelu": lambda: torch.nn.functional.gelu(f, approximate="tanh"),
        "gelu_erf": lambda: torch.nn.functional.gelu(f), "inv_sqrt": lambda: torch.rsqrt(f + a),
        "pow": lambda: f.pow(a), "clamp": lambda: f.clamp(a, b),
        "leaky_relu": lambda: torch.nn.functional.leaky_relu(f, a), "neg": lambda: -f,
        "reciprocal": lambda: f.reciprocal(),
    }[name]()
    return out.to(x.dtype)


def binary_reference(name: str, x: torch.Tensor, y: torch.Tensor, a: float = 1.0, b: float = 1.0) -> torch.Tensor:
    f, g = x.float(), y.float()
    out = {"add": lambda: f + g, "sub": lambda: f - g, "mul": lambda: f * g, "div": lambda: f / g,
           "max": lambda: torch.maximum(f, g), "min": lambda: torch.minimum(f, g),
           "axpby": lambda: a * f + b * g}[name]()
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------------------------- raw launchers
def _unary_raw(name, x, a, b):
    x = _c(x)
    y = torch.empty_like(x)
    rc = _native.lib().idrak_pw_unary(UNARY[name], _DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), x.numel(), float(a),
                                      float(b), stream_ptr())
    _native.check(rc, f"idrak_pw_unary({name})")
    return y


def _unary_bwd_raw(name, x, dy, a, b, into=None):
    x, dy = _c(x), _c(dy)
    dx = into if into is not None else torch.empty_like(x)
    rc = _native.lib().idrak_pw_unary_bwd(UNARY[name], _DTYPES[x.dtype], x.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                          x.numel(), float(a), float(b), int(into is not None), stream_ptr())
    _native.check(rc, f"idrak_pw_unary_bwd({name})")
    return dx


def _binary_raw(name, x, y, a=1.0, b=1.0):
    x, y = _c(x), _c(y)
    out = torch.empty_like(x)
    rc = _native.lib().idrak_pw_binary(BINARY[name], _DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), out.data_ptr(),
                                       x.numel(), float(a), float(b), stream_ptr())
    _native.check(rc, f"idrak_pw_binary({name})")
    return out


class _Unary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name, a, b):
        ctx.save_for_backward(x)
        ctx.spec = (name, a, b)
        return _unary_raw(name, x, a, b)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        name, a, b = ctx.spec
        return _unary_bwd_raw(name, x, dy, a, b), None, None, None


def unary(name: str, x: torch.Tensor, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
    """``f(x)`` for a name of ``UNARY``; ``a`` / ``b`` are the function's constants (slope and offset of ``affine``,
    the exponent of ``pow``, the bounds of ``clamp``, the negative slope of ``leaky_relu``, the epsilon of
    ``inv_sqrt``)."""
    if name not in UNARY:
        raise KeyError(f"unknown unary operation '{name}'. Known: {', '.join(UNARY)}")
    if not _native_ok(x):
        return unary_reference(name, x, a, b)
    return _Unary.apply(x, name, float(a), float(b))


def unary_backward(name: str, x: torch.Tensor, dy: torch.Tensor, a: float = 0.0, b: float = 0.0,
                   accumulate_into: torch.Tensor | None = None) -> torch.Tensor:
    """``dy * f'(x)``, written to a new tensor or added to ``accumulate_into``."""
    if not _native_ok(x, dy):
        xs = x.detach().float().requires_grad_(True)
        with torch.enable_grad():
            unary_reference(name, xs, a, b).backward(dy.float())
        g = xs.grad.to(x.dtype)
        if accumulate_into is not None:
            accumulate_into.add_(g)
            return accumulate_into
        return g
    return _unary_bwd_raw(name, x, dy, a, b, accumulate_into)


class _Binary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, name, a, b):
        ctx.save_for_backward(x, y)
        ctx.spec = (name, a, b)
        return _binary_raw(name, x, y, a, b)

    @staticmethod
    def backward(ctx, dy):
        x, y = ctx.saved_tensors
        name, a, b = ctx.spec
        dy = _c(dy)
        if name == "add":
            return dy, dy, None, None, None
        if name == "sub":
            return dy, _unary_raw("neg", dy, 0, 0), None, None, None
        if name == "axpby":
            return _unary_raw("affine", dy, a, 0), _unary_raw("affine", dy, b, 0), None, None, None
        if name == "mul":
            return _binary_raw("mul", dy, y), _binary_raw("mul", dy, x), None, None, None
        if name == "div":
            q = _binary_raw("div", dy, y)                                   # dy / y
            return q, _unary_raw("neg", _binary_raw("mul", q, _binary_raw("div", x, y)), 0, 0), None, None, None
        dx, dyo = torch.empty_like(x), torch.empty_like(x)
        rc = _native.lib().idrak_pw_extremum_bwd(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                                 dx.data_ptr(), dyo.data_ptr(), x.numel(), int(name == "max"),
                                                 stream_ptr())
        _native.check(rc, "idrak_pw_extremum_bwd")
        return dx, dyo, None, None, None


def binary(name: str, x: torch.Tensor, y: torch.Tensor, a: float = 1.0, b: float = 1.0) -> torch.Tensor:
    """``x (op) y`` for same-shaped operands; ``axpby`` is ``a * x + b * y``. On a tie ``max`` / ``min`` send the whole
    gradient to ``x``."""
    if name not in BINARY:
        raise KeyError(f"unknown binary operation '{name}'. Known: {', '.join(BINARY)}")
    if not _native_ok(x, y):
        return binary_reference(name, x, y, a, b)
    return _Binary.apply(_c(x), _c(y), name, float(a), float(b))


class _MulAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, z):
        ctx.save_for_backward(x, y)
        out = torch.empty_like(x)
        rc = _native.lib().idrak_pw_muladd(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), z.data_ptr(), out.data_ptr(),
                                           x.numel(), stream_ptr())
        _native.check(rc, "idrak_pw_muladd")
        return out

    @staticmethod
    def backward(ctx, dy):
        x, y = ctx.saved_tensors
        dy = _c(dy)
        return _binary_raw("mul", dy, y), _binary_raw("mul", dy, x), dy


def muladd(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """``x * y + z`` in one pass."""
    if not _native_ok(x, y, z):
        return (x.float() * y.float() + z.float()).to(x.dtype)
    return _MulAdd.apply(_c(x), _c(y), _c(z))


class _Where(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cond, x, y):
        ctx.save_for_backward(cond)
        return _where_raw(cond, x, y)

    @staticmethod
    def backward(ctx, dy):
        (cond,) = ctx.saved_tensors
        zero = torch.zeros_like(dy)
        dy = _c(dy)
        return None, _where_raw(cond, dy, zero), _where_raw(cond, zero, dy)


def _where_raw(cond, x, y):
    out = torch.empty_like(x)
    rc = _native.lib().idrak_pw_where(_DTYPES[x.dtype], cond.data_ptr(), x.data_ptr(), y.data_ptr(), out.data_ptr(),
                                      x.numel(), stream_ptr())
    _native.check(rc, "idrak_pw_where")
    return out


def where(cond: torch.Tensor, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``cond ? x : y`` (``cond``: bool or uint8 of the same shape)."""
    if not (_native_ok(x, y) and cond.is_cuda and cond.shape == x.shape and cond.dtype in (torch.bool, torch.uint8)):
        return torch.where(cond.bool(), x, y)
    c8 = _c(cond).view(torch.uint8) if cond.dtype == torch.bool else _c(cond)
    return _Where.apply(c8, _c(x), _c(y))


def fill_(t: torch.Tensor, value: float) -> torch.Tensor:
    if not (_native_ok(t) and t.is_contiguous()):
        return t.fill_(value)
    rc = _native.lib().idrak_pw_fill(_DTYPES[t.dtype], t.data_ptr(), t.numel(), float(value), stream_ptr())
    _native.check(rc, "idrak_pw_fill")
    return t


class _AddRowVec(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, vec):
        out = torch.empty_like(x)
        cols = x.shape[-1]
        rc = _native.lib().idrak_pw_add_rowvec(_DTYPES[x.dtype], x.data_ptr(), vec.data_ptr(), out.data_ptr(),
                                               x.numel() // cols, cols, stream_ptr())
        _native.check(rc, "idrak_pw_add_rowvec")
        return out

    @staticmethod
    def backward(ctx, dy):
        from .reduce import sum_axis
        cols = dy.shape[-1]
        return dy, sum_axis(dy.reshape(-1, cols), 0).to(dy.dtype)


def add_rowvec(x: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """``x[..., c] + vec[c]`` (a bias add)."""
    cols = x.shape[-1]
    ok = (_native_ok(x) and vec.is_cuda and vec.dtype == x.dtype and vec.numel() == cols
          and cols % (4 if x.dtype == torch.float32 else 8) == 0)
    if not ok:
        return (x.float() + vec.float()).to(x.dtype)
    return _AddRowVec.apply(_c(x), _c(vec))


# ------------------------------------------------------------------------------------------------------------- dropout
_MASK64 = (1 << 64) - 1


def uniform_reference(seed: int, n: int) -> torch.Tensor:
    """The generator the dropout kernel draws from, on the host: element i of a call with this seed."""
    out = torch.empty(n, dtype=torch.float32)
    for i in range(n):
        z = (seed + (i + 1) * 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        z ^= z >> 31
        out[i] = (z >> 40) / 16777216.0
    return out


def dropout_reference(x, p, seed, residual=None):
    keep = (uniform_reference(seed, x.numel()).reshape(x.shape) >= p).to(x.device)
    out = x.float() * keep / (1.0 - p)
    if residual is not None:
        out = out + residual.float()
    return out.to(x.dtype)


def _dropout_raw(x, residual, p, seed):
    out = torch.empty_like(x)
    rc = _native.lib().idrak_pw_dropout(_DTYPES[x.dtype], x.data_ptr(), ptr(residual), out.data_ptr(), x.numel(),
                                        float(p), int(seed) & _MASK64, stream_ptr())
    _native.check(rc, "idrak_pw_dropout")
    return out


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, seed):
        ctx.spec = (p, seed, residual is not None)
        return _dropout_raw(x, residual, p, seed)

    @staticmethod
    def backward(ctx, dy):
        p, seed, has_res = ctx.spec
        dy = _c(dy)
        return _dropout_raw(dy, None, p, seed), (dy if has_res else None), None, None


def dropout(x: torch.Tensor, p: float, seed: int, residual: torch.Tensor | None = None,
            training: bool = True) -> torch.Tensor:
    """``residual + keep * x / (1 - p)`` where ``keep`` is drawn per element from (seed, element index); no mask is
    stored, the backward pass draws it again. With ``training=False`` (or p = 0) it is the identity (plus residual)."""
    if not 0.0 <= p < 1.0:
        raise ValueError(f"dropout probability must be in [0, 1), got {p}")
    if not training or p == 0.0:
        return x if residual is None else binary("add", x, residual)
    ts = (x,) if residual is None else (x, residual)
    if not _native_ok(*ts):
        if x.numel() > 1 << 16:                      # the host statement of the generator is a Python loop
            keep = (torch.rand(x.shape, generator=torch.Generator().manual_seed(seed & 0x7FFFFFFF)) >= p).to(x.device)
            out = x * keep / (1.0 - p)
            return out if residual is None else out + residual
        return dropout_reference(x, p, seed, residual)
    return _Dropout.apply(_c(x), None if residual is None else _c(residual), float(p), int(seed))


def _make(name):
    def f(x: torch.Tensor) -> torch.Tensor:
        return unary(name, x)
    f.__name__ = name
    f.__doc__ = f"Element-wise {name} with its gradient."
    return f


sigmoid, tanh, relu, square, absolute, sqrt, sin, cos, silu, sign, exp, log, gelu_erf, neg, reciprocal = (
    _make(n) for n in ("sigmoid", "tanh", "relu", "square", "abs", "sqrt", "sin", "cos", "silu", "sign", "exp", "log",
                       "gelu_erf", "neg", "reciprocal"))


def affine(x, scale: float, offset: float = 0.0):
    return unary("affine", x, scale, offset)


def add_scalar(x, value: float):
    return unary("affine", x, 1.0, value)


def power(x, exponent: float):
    return unary("pow", x, exponent)


def clamp(x, low: float = -math.inf, high: float = math.inf):
    return unary("clamp", x, max(low, -3.0e38), min(high, 3.0e38))


def leaky_relu(x, slope: float = 0.01):
    return unary("leaky_relu", x, slope)


def inv_sqrt(x, eps: float = 0.0):
    return unary("inv_sqrt", x, eps)


def sub(x, y):
    return binary("sub", x, y)


def mul(x, y):
    return binary("mul", x, y)


def div(x, y):
    return binary("div", x, y)


def maximum(x, y):
    return binary("max", x, y)


def minimum(x, y):
    return binary("min", x, y)


def axpby(a: float, x, b: float, y):
    return binary("axpby", x, y, a, b)
