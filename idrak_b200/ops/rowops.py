"""Row-wise and element-wise ops: LayerNorm / RMSNorm, GELU, gated activations, RoPE, embedding,
column sums. CUDA bf16 tensors run the sm_100a kernels; CPU tensors run plain PyTorch.

Reference: Tensor.LayerNormTrain (src/Idrak.Abstraction/Tensors/Tensor.Decoding.cs:53),
Tensor.RmsNormAffine / Rope (Tensor.Decoder.cs:370,523), GatedActivation, EmbeddingLookup.
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, scratch, stream_ptr

GATE_KINDS = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "relu": 2, "reglu": 2, "tanh": 3}


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


# --------------------------------------------------------------------------- column sums
def colsum(x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Sum over rows of a 2-D bf16 matrix (the bias gradient)."""
    if not _native_ok(x):
        s = x.float().sum(0)
        if out is not None:
            out.copy_((out.float() + s if accumulate else s).to(out.dtype))
            return out
        return s.to(x.dtype)
    rows, C = x.shape
    assert x.stride(1) == 1
    lib = _native.lib()
    if out is None:
        out = torch.empty(C, dtype=x.dtype, device=x.device)
    part = scratch("colsum", lib.idrak_colsum_blocks(rows) * C, torch.float32, x.device)
    rc = lib.idrak_colsum(x.data_ptr(), rows, C, x.stride(0), part.data_ptr(), out.data_ptr(),
                          1 if out.dtype == torch.float32 else 0, int(accumulate), stream_ptr())
    _native.check(rc, "idrak_colsum")
    return out


# --------------------------------------------------------------------------- norms
def norm_forward(x, weight, bias, eps, rms, residual=None):
    """Returns (out, mean, rstd, summed) where summed = x + residual when residual is given."""
    C = x.shape[-1]
    x2 = x.reshape(-1, C)
    rows = x2.shape[0]
    if not _native_ok(x):
        xs = x2.float() + (residual.reshape(-1, C).float() if residual is not None else 0)
        summed = xs.to(x.dtype) if residual is not None else None
        xf = summed.float() if summed is not None else xs
        if rms:
            mean = torch.zeros(rows, device=x.device)
            rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
            out = xf * rstd[:, None] * weight.float()
        else:
            mean = xf.mean(-1)
            var = xf.var(-1, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            out = (xf - mean[:, None]) * rstd[:, None] * weight.float()
            if bias is not None:
                out = out + bias.float()
        return (out.to(x.dtype).reshape(x.shape), mean, rstd,
                summed.reshape(x.shape) if summed is not None else None)
    x2 = x2.contiguous()
    out = torch.empty_like(x2)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    r2 = residual.reshape(-1, C).contiguous() if residual is not None else None
    summed = torch.empty_like(x2) if residual is not None else None
    rc = _native.lib().idrak_norm_fwd(x2.data_ptr(), ptr(r2), weight.data_ptr(), ptr(bias), out.data_ptr(),
                                      ptr(summed), mean.data_ptr(), rstd.data_ptr(), rows, C, float(eps),
                                      int(rms), stream_ptr())
    _native.check(rc, "idrak_norm_fwd")
    return out.reshape(x.shape), mean, rstd, (summed.reshape(x.shape) if summed is not None else None)


def norm_backward(dy, x, weight, mean, rstd, rms, has_bias, dres=None, w_param=None, b_param=None,
                  sums_of_dx: bool = False):
    """Returns (dx, dweight, dbias). ``x`` is the tensor that was normalised. ``dres`` is added to dx.
    When ``w_param`` (and ``b_param``) take direct gradient writes, dweight / dbias go straight into their
    ``.grad`` and come back as None. With ``sums_of_dx`` the column sums of dx (fp32) are attached to the returned
    dx as ``_idrak_colsum`` where the kernel produces them on the way (rows of up to 1024 elements): dx is the
    output gradient of the linear layer before this norm, so ``ops.gemm.bias_grad`` finds its bias gradient there."""
    C = x.shape[-1]
    dy2, x2 = dy.reshape(-1, C), x.reshape(-1, C)
    rows = x2.shape[0]
    if not _native_ok(x):
        xf, g = x2.float(), dy2.float()
        n = (xf - (0 if rms else mean[:, None])) * rstd[:, None]
        gw = g * weight.float()
        s2 = (gw * n).mean(-1, keepdim=True)
        s1 = 0 if rms else gw.mean(-1, keepdim=True)
        dx = (gw - s1 - n * s2) * rstd[:, None]
        if dres is not None:
            dx = dx + dres.reshape(-1, C).float()
        dw = (g * n).sum(0)
        db = g.sum(0) if has_bias else None
        return dx.to(x.dtype).reshape(x.shape), dw.to(weight.dtype), (db.to(weight.dtype) if has_bias else None)
    lib = _native.lib()
    dy2, x2 = dy2.contiguous(), x2.contiguous()
    dx = torch.empty_like(x2)
    blocks = lib.idrak_norm_bwd_blocks(rows)
    part = scratch("norm_bwd", 3 * blocks * C, torch.float32, x.device)
    from . import _grad
    tw = _grad.target(w_param)
    tb = _grad.target(b_param) if has_bias else None
    direct = tw is not None and (not has_bias or tb is not None)
    if direct:
        dw, accumulate = tw
        db = tb[0] if has_bias else None
    else:
        dw, accumulate = torch.empty_like(weight), False
        db = torch.empty_like(weight) if has_bias else None
    d2 = dres.reshape(-1, C).contiguous() if dres is not None else None
    sums = None
    if sums_of_dx and lib.idrak_norm_bwd_sums_dx(rows, C):
        sums = torch.empty(C, dtype=torch.float32, device=x.device)
    rc = lib.idrak_norm_bwd_fused(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(), ptr(mean), rstd.data_ptr(), ptr(d2),
                                  dx.data_ptr(), part.data_ptr(), dw.data_ptr(), ptr(db), ptr(sums),
                                  1 if dw.dtype == torch.float32 else 0, int(accumulate), rows, C, int(rms),
                                  stream_ptr())
    _native.check(rc, "idrak_norm_bwd_fused")
    dx = dx.reshape(x.shape)
    if sums is not None:
        dx._idrak_colsum = (sums, dx._version)      # the version guards against a later in-place accumulation
    if direct:
        _grad.written(w_param)
        if has_bias:
            _grad.written(b_param)
        return dx, None, None
    return dx, dw, db


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        out, mean, rstd, _ = norm_forward(x, weight, bias, eps, rms)
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.params = (weight, bias)
        ctx.rms, ctx.has_bias = rms, bias is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dx, dw, db = norm_backward(dy, x, weight, mean, rstd, ctx.rms, ctx.has_bias, None, *ctx.params)
        return dx, dw, db, None, None


class _NormBranch(torch.autograd.Function):
    """``(norm(x), x)``: the second output is the residual path of a pre-norm block. Both gradients arrive in one
    backward call, so the residual gradient is added inside the norm-backward kernel (no separate add) and the
    column sums of the joint gradient come out of the same pass."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        out, mean, rstd, _ = norm_forward(x, weight, bias, eps, rms)
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.params = (weight, bias)
        ctx.rms, ctx.has_bias = rms, bias is not None
        return out, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x, weight, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None, None
        dx, dw, db = norm_backward(dy, x, weight, mean, rstd, ctx.rms, ctx.has_bias, dres, *ctx.params,
                                   sums_of_dx=True)
        return dx, dw, db, None, None


def norm_branch(x, weight, bias=None, eps: float = 1e-5, rms: bool = False):
    """``(norm(x), x)`` for a pre-norm residual block: feed the first to the sub-layer and the second to its
    residual input. Equal to computing the norm and reusing ``x``; on the GPU the backward pass is one kernel."""
    if not _native_ok(x):
        if rms:
            return rms_norm(x, weight, eps), x
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps), x
    return _NormBranch.apply(x, weight, bias, eps, rms)


def layer_norm(x, weight, bias=None, eps: float = 1e-5):
    if not _native_ok(x):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    return _Norm.apply(x, weight, bias, eps, False)


def rms_norm(x, weight, eps: float = 1e-5):
    if not _native_ok(x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)
    return _Norm.apply(x, weight, None, eps, True)


# --------------------------------------------------------------------------- activations
class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        _native.check(_native.lib().idrak_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), stream_ptr()), "gelu_fwd")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        _native.check(_native.lib().idrak_gelu_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(),
                                                   stream_ptr()), "gelu_bwd")
        return dx


def gelu(x):
    """GELU, tanh form."""
    if not _native_ok(x) or x.numel() % 8:
        return torch.nn.functional.gelu(x, approximate="tanh")
    return _Gelu.apply(x)


def _gate_ref(g, kind):
    if kind == 0:
        return torch.nn.functional.silu(g)
    if kind == 1:
        return torch.nn.functional.gelu(g, approximate="tanh")
    if kind == 2:
        return torch.relu(g)
    return torch.tanh(g)


class _Gated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, kind):
        H = gu.shape[-1] // 2
        gu2 = gu.reshape(-1, 2 * H).contiguous()
        out = torch.empty((gu2.shape[0], H), dtype=gu.dtype, device=gu.device)
        _native.check(_native.lib().idrak_gated_fwd(gu2.data_ptr(), out.data_ptr(), gu2.shape[0], H, kind,
                                                    stream_ptr()), "gated_fwd")
        ctx.save_for_backward(gu2)
        ctx.kind, ctx.shape = kind, gu.shape
        return out.reshape(*gu.shape[:-1], H)

    @staticmethod
    def backward(ctx, dout):
        (gu2,) = ctx.saved_tensors
        H = gu2.shape[1] // 2
        d2 = dout.reshape(-1, H).contiguous()
        dgu = torch.empty_like(gu2)
        _native.check(_native.lib().idrak_gated_bwd(gu2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), gu2.shape[0], H,
                                                    ctx.kind, stream_ptr()), "gated_bwd")
        return dgu.reshape(ctx.shape), None


def gated_activation(gate_up: torch.Tensor, kind: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` with gate = first half of the last dim, up = second half."""
    k = GATE_KINDS[kind]
    H = gate_up.shape[-1] // 2
    if not _native_ok(gate_up) or H % 8:
        g, u = gate_up[..., :H], gate_up[..., H:]
        return _gate_ref(g, k) * u
    return _Gated.apply(gate_up, k)


# --------------------------------------------------------------------------- RoPE
def rope_reference(x, positions, theta, rot_dim=None, freq_scale=1.0, inverse=False):
    """x: [tokens, heads, D]; rotate-half pairs (i, i + rot/2)."""
    D = x.shape[-1]
    rot = rot_dim or D
    half = rot // 2
    k = torch.arange(half, device=x.device, dtype=torch.float32)
    inv_freq = theta ** (-2.0 * k / rot)
    ang = positions.float()[:, None] * freq_scale * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if inverse:
        s = -s
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rot] = b * c + a * s
    return out.to(x.dtype)


def rope_(x: torch.Tensor, positions: torch.Tensor | None, theta: float, rot_dim: int | None = None,
          freq_scale: float = 1.0, inverse: bool = False) -> torch.Tensor:
    """In-place rotary embedding on a [tokens, heads, D] view whose last two dims are contiguous."""
    tokens, heads, D = x.shape
    if not _native_ok(x):
        pos = positions if positions is not None else torch.arange(tokens, device=x.device)
        x.copy_(rope_reference(x, pos, theta, rot_dim, freq_scale, inverse))
        return x
    assert x.stride(2) == 1 and x.stride(1) == D
    if positions is not None:
        assert positions.dtype == torch.int32 and positions.is_contiguous()
    rc = _native.lib().idrak_rope(x.data_ptr(), ptr(positions), tokens, heads, D, x.stride(0), rot_dim or D,
                                  float(theta), float(freq_scale), int(inverse), stream_ptr())
    _native.check(rc, "idrak_rope")
    return x


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, theta, rot_dim, freq_scale):
        y = x.clone()
        rope_(y, positions, theta, rot_dim, freq_scale, False)
        ctx.positions, ctx.args = positions, (theta, rot_dim, freq_scale)
        return y

    @staticmethod
    def backward(ctx, dy):
        d = dy.clone()
        theta, rot_dim, freq_scale = ctx.args
        rope_(d, ctx.positions, theta, rot_dim, freq_scale, True)
        return d, None, None, None, None


def rope(x, positions, theta=10000.0, rot_dim=None, freq_scale=1.0):
    return _Rope.apply(x, positions, theta, rot_dim, freq_scale)


# --------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, seq):
        tokens = ids.numel()
        C = wte.shape[1]
        ids32 = ids.reshape(-1).to(torch.int32).contiguous()
        out = torch.empty((tokens, C), dtype=wte.dtype, device=wte.device)
        rc = _native.lib().idrak_embedding_fwd(ids32.data_ptr(), wte.data_ptr(), ptr(wpe), out.data_ptr(), tokens,
                                               seq, C, stream_ptr())
        _native.check(rc, "idrak_embedding_fwd")
        ctx.save_for_backward(ids32)
        ctx.params = (wte, wpe)
        ctx.wte_shape, ctx.wpe_shape, ctx.seq = wte.shape, (wpe.shape if wpe is not None else None), seq
        ctx.dtype = wte.dtype
        return out.reshape(*ids.shape, C)

    @staticmethod
    def backward(ctx, dout):
        (ids32,) = ctx.saved_tensors
        C = ctx.wte_shape[1]
        d2 = dout.reshape(-1, C).contiguous()
        tokens = d2.shape[0]
        lib = _native.lib()
        from . import _grad
        p_wte, p_wpe = ctx.params
        tgt = _grad.target(p_wte)
        if tgt is not None:
            dwte, accumulate = tgt
            if not accumulate:
                dwte.zero_()          # the kernel adds the rows of the tokens that occur
        else:
            dwte = torch.zeros(ctx.wte_shape, dtype=ctx.dtype, device=dout.device)
        sorted_ids, order = torch.sort(ids32, stable=True)
        order32 = order.to(torch.int32)
        rc = lib.idrak_wte_bwd(sorted_ids.data_ptr(), order32.data_ptr(), d2.data_ptr(), dwte.data_ptr(), tokens, C,
                               1 if dwte.dtype == torch.float32 else 0, stream_ptr())
        _native.check(rc, "idrak_wte_bwd")
        if tgt is not None:
            _grad.written(p_wte)
            dwte = None
        dwpe = None
        if ctx.wpe_shape is not None:
            tp = _grad.target(p_wpe)
            if tp is not None:
                g, accumulate = tp
                rc = lib.idrak_wpe_bwd(d2.data_ptr(), g.data_ptr(), tokens // ctx.seq, ctx.seq, C,
                                       1 if g.dtype == torch.float32 else 0, int(accumulate), stream_ptr())
                _native.check(rc, "idrak_wpe_bwd")
                _grad.written(p_wpe)
            else:
                dwpe = torch.zeros(ctx.wpe_shape, dtype=ctx.dtype, device=dout.device)
                rc = lib.idrak_wpe_bwd(d2.data_ptr(), dwpe.data_ptr(), tokens // ctx.seq, ctx.seq, C, 0, 0,
                                       stream_ptr())
                _native.check(rc, "idrak_wpe_bwd")
        return None, dwte, dwpe, None


def embedding(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor | None = None) -> torch.Tensor:
    """``wte[ids] (+ wpe[position])``; ids is [batch, seq]."""
    seq = ids.shape[-1]
    if not _native_ok(wte) or wte.shape[1] % 8:
        out = torch.nn.functional.embedding(ids.long(), wte)
        if wpe is not None:
            out = out + wpe[:seq]
        return out
    return _Embedding.apply(ids, wte, wpe, seq)


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a + b
