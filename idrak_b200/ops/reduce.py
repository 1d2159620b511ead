"""Softmax family, axis sums, permutation and index operations. CUDA fp32 / bf16 tensors run ``csrc/reduce_ops.cu``;
other tensors run the plain PyTorch statement, which is the test oracle as well.

Reference: Tensor.Softmax / LogSoftmax / ScaleMaskSoftmax / Sum(axis) / Permute / Transpose / Gather / OneHot
(src/Idrak.Abstraction/Tensors/Tensor.cs, Tensor.Decoding.cs) and softmax_f32, softmax_bwd, scale_mask_softmax_f32,
sum_axis, broadcast_axis, permute, gather_f32, one_hot, class_match (src/Idrak.Gpu/Cuda/PtxKernels.Advanced.cs:12,
PtxKernels.Decoding.cs:12).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native
from ._util import ptr, stream_ptr

_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def _ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in _DTYPES and t.numel() > 0


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


# ------------------------------------------------------------------------------------------------------------- softmax
def softmax_reference(x, scale=1.0, mask=None, causal=False, log=False):
    s = x.float() * scale
    tq, tk = (x.shape[-2], x.shape[-1]) if x.dim() >= 2 else (1, x.shape[-1])
    if mask is not None:
        s = s + mask.float()
    if causal:
        keep = torch.ones(tq, tk, dtype=torch.bool, device=x.device).tril(tk - tq)
        s = s.masked_fill(~keep, float("-inf"))
    out = torch.log_softmax(s, -1) if log else torch.softmax(s, -1)
    return torch.nan_to_num(out, nan=0.0, neginf=-3.4028234663852886e38 if log else 0.0).to(x.dtype)


def _softmax_raw(x, scale, mask, causal, log):
    cols = x.shape[-1]
    rows = x.numel() // cols
    tq = x.shape[-2] if x.dim() >= 2 else 1
    y = torch.empty_like(x)
    mask_rows = 0
    if mask is not None:
        mask_rows = mask.numel() // cols
    rc = _native.lib().idrak_softmax(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), rows, cols, float(scale), ptr(mask),
                                     mask_rows, int(causal), tq, cols - tq, int(log), stream_ptr())
    _native.check(rc, "idrak_softmax")
    return y


class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, mask, causal, log):
        y = _softmax_raw(x, scale, mask, causal, log)
        ctx.save_for_backward(y)
        ctx.spec = (scale, log)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        scale, log = ctx.spec
        dy = _c(dy)
        dx = torch.empty_like(y)
        cols = y.shape[-1]
        rc = _native.lib().idrak_softmax_bwd(_DTYPES[y.dtype], y.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                             y.numel() // cols, cols, float(scale), int(log), stream_ptr())
        _native.check(rc, "idrak_softmax_bwd")
        return dx, None, None, None, None


def softmax(x: torch.Tensor, dim: int = -1, *, scale: float = 1.0, mask: torch.Tensor | None = None,
            causal: bool = False, log: bool = False) -> torch.Tensor:
    """Softmax (or log-softmax) of ``scale * x + mask`` over ``dim``. ``mask``: additive, fp32, shaped
    ``[..., rows, cols]`` with as many leading rows as it wants to cover (row r of ``x`` uses mask row
    ``r % mask_rows``, so a ``[Tq, Tk]`` mask serves every batch and head). ``causal`` keeps column c of query row q
    (the second-to-last axis) when ``c <= q + (Tk - Tq)``. A fully masked row gives zeros."""
    if dim not in (-1, x.dim() - 1):
        return softmax(x.transpose(dim, -1), -1, scale=scale, mask=mask, causal=causal, log=log).transpose(dim, -1)
    if mask is not None and mask.shape[-1] != x.shape[-1]:
        raise ValueError(f"mask has {mask.shape[-1]} columns, the scores {x.shape[-1]}")
    if not _ok(x):
        return softmax_reference(x, scale, mask, causal, log)
    m = None
    if mask is not None:
        m = mask.to(device=x.device, dtype=torch.float32)
        if x.dim() >= 2 and tuple(m.shape) != tuple(x.shape[-2:]) and m.numel() != x.numel():
            m = m.expand(x.shape)                     # any other broadcast: materialise it once
        m = _c(m)
    return _Softmax.apply(_c(x), float(scale), m, bool(causal), bool(log))


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return softmax(x, dim, log=True)


def scale_mask_softmax(scores: torch.Tensor, scale: float, mask: torch.Tensor | None = None,
                       causal: bool = True) -> torch.Tensor:
    """Attention probabilities from raw scores ``[..., Tq, Tk]`` in one pass."""
    return softmax(scores, -1, scale=scale, mask=mask, causal=causal)


# ----------------------------------------------------------------------------------------------------------- axis sums
def sum_axis(x: torch.Tensor, axis: int, scale: float = 1.0) -> torch.Tensor:
    """Sum over one axis in fp32 (``scale`` folds a mean in). The result drops the axis."""
    axis = axis % x.dim()
    if not _ok(x):
        return x.float().sum(axis) * scale
    x = _c(x)
    outer = 1
    for s in x.shape[:axis]:
        outer *= s
    inner = x.numel() // (outer * x.shape[axis])
    out = torch.empty(x.shape[:axis] + x.shape[axis + 1:], dtype=torch.float32, device=x.device)
    rc = _native.lib().idrak_sum_axis(_DTYPES[x.dtype], x.data_ptr(), out.data_ptr(), outer, x.shape[axis], inner,
                                      float(scale), stream_ptr())
    _native.check(rc, "idrak_sum_axis")
    return out


def broadcast_axis(x: torch.Tensor, axis: int, size: int, dtype: torch.dtype | None = None,
                   accumulate_into: torch.Tensor | None = None) -> torch.Tensor:
    """The inverse of ``sum_axis``: repeat an fp32 tensor ``size`` times along a new axis (or add it into a tensor of
    that shape): the gradient of a sum, the forward of a broadcast."""
    axis = axis % (x.dim() + 1)
    shape = tuple(x.shape[:axis]) + (size,) + tuple(x.shape[axis:])
    out = accumulate_into
    dtype = dtype or (out.dtype if out is not None else torch.float32)
    if not (x.is_cuda and x.dtype == torch.float32 and dtype in _DTYPES and x.numel() > 0):
        rep = x.float().unsqueeze(axis).expand(shape)
        if out is not None:
            out.add_(rep.to(out.dtype))
            return out
        return rep.to(dtype).contiguous()
    x = _c(x)
    if out is None:
        out = torch.empty(shape, dtype=dtype, device=x.device)
    assert out.is_contiguous() and tuple(out.shape) == shape
    outer = 1
    for s in x.shape[:axis]:
        outer *= s
    inner = x.numel() // outer
    rc = _native.lib().idrak_broadcast_axis(_DTYPES[out.dtype], x.data_ptr(), out.data_ptr(), outer, size, inner,
                                            int(accumulate_into is not None), stream_ptr())
    _native.check(rc, "idrak_broadcast_axis")
    return out


# --------------------------------------------------------------------------------------------------- layout operations
def permute(x: torch.Tensor, order) -> torch.Tensor:
    """A contiguous copy with the axes in ``order`` (rank up to six; a swap of the two innermost axes takes the tiled
    path)."""
    order = [o % x.dim() for o in order]
    if sorted(order) != list(range(x.dim())):
        raise ValueError(f"{order} is not a permutation of {x.dim()} axes")
    if not _ok(x) or x.dim() > 6 or x.dim() < 2:
        return x.permute(order).contiguous()
    x = _c(x)
    lib = _native.lib()
    n = x.dim()
    if order == list(range(n - 2)) + [n - 1, n - 2]:
        rows, cols = x.shape[-2], x.shape[-1]
        batch = x.numel() // (rows * cols)
        if batch <= 65535:
            y = torch.empty(x.shape[:-2] + (cols, rows), dtype=x.dtype, device=x.device)
            rc = lib.idrak_transpose(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), batch, rows, cols, stream_ptr())
            _native.check(rc, "idrak_transpose")
            return y
    out_dims = [x.shape[o] for o in order]
    src_strides = [x.stride(o) for o in order]
    y = torch.empty(out_dims, dtype=x.dtype, device=x.device)
    arr = C.c_longlong * n
    rc = lib.idrak_permute(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), n, arr(*out_dims), arr(*src_strides),
                           stream_ptr())
    _native.check(rc, "idrak_permute")
    return y


def transpose(x: torch.Tensor) -> torch.Tensor:
    """Swap the two innermost axes (contiguous result)."""
    return permute(x, list(range(x.dim() - 2)) + [x.dim() - 1, x.dim() - 2])


def gather_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """``table[ids]`` for a 2-D table; an id outside the table gives a row of zeros."""
    if not (_ok(table) and table.dim() == 2 and ids.is_cuda):
        safe = ids.clamp(0, table.shape[0] - 1)
        out = table[safe]
        bad = (ids < 0) | (ids >= table.shape[0])
        return out.masked_fill(bad.unsqueeze(-1), 0)
    table = _c(table)
    flat = _c(ids.reshape(-1).to(torch.int32))
    out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    rc = _native.lib().idrak_gather_rows(_DTYPES[table.dtype], table.data_ptr(), flat.data_ptr(), out.data_ptr(),
                                         flat.numel(), table.shape[1], table.shape[0], stream_ptr())
    _native.check(rc, "idrak_gather_rows")
    return out.reshape(tuple(ids.shape) + (table.shape[1],))


def one_hot(ids: torch.Tensor, classes: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if not (ids.is_cuda and dtype in _DTYPES and ids.numel() > 0):
        return torch.nn.functional.one_hot(ids.long().clamp(0, classes - 1), classes).to(dtype) * \
            ((ids >= 0) & (ids < classes)).unsqueeze(-1).to(dtype)
    flat = _c(ids.reshape(-1).to(torch.int32))
    out = torch.empty((flat.numel(), classes), dtype=dtype, device=ids.device)
    rc = _native.lib().idrak_one_hot(_DTYPES[dtype], flat.data_ptr(), out.data_ptr(), flat.numel(), classes,
                                     stream_ptr())
    _native.check(rc, "idrak_one_hot")
    return out.reshape(tuple(ids.shape) + (classes,))


def class_match(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """How many rows have their arg-max (lowest index on a tie) at the target; rows with a negative target are left
    out. Returns a 0-d int32 tensor on the device of ``logits`` (no host read)."""
    cols = logits.shape[-1]
    if not _ok(logits):
        l2, t = logits.reshape(-1, cols).float(), targets.reshape(-1)
        return ((l2.argmax(-1) == t) & (t >= 0)).sum().to(torch.int32)
    l2 = _c(logits).reshape(-1, cols)
    t = _c(targets.reshape(-1).to(torch.int32))
    count = torch.zeros((), dtype=torch.int32, device=logits.device)
    rc = _native.lib().idrak_class_match(_DTYPES[l2.dtype], l2.data_ptr(), t.data_ptr(), l2.shape[0], cols,
                                         count.data_ptr(), stream_ptr())
    _native.check(rc, "idrak_class_match")
    return count
