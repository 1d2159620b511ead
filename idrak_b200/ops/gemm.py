"""Dense GEMM on the tcgen05 kernel, and the ``Linear`` autograd function built on it.

``gemm`` exposes the kernel's full contract (operand majors, fused epilogue, split-K).
``linear`` is the layer-level entry: ``y = act(x @ W^T + b) (+ residual)`` with a backward pass that
runs the input gradient (K-major x MN-major) and the weight gradient (MN-major x MN-major, split-K) on
the same kernel, so no transposed copy of an activation or a weight is ever made.

On CPU tensors the same functions compute in plain PyTorch (fp32 for config-1-style CPU runs and as
the oracle the GPU tests compare against).

Reference: Tensor.MatMul (src/Idrak.Abstraction/Tensors/Tensor.Advanced.cs:31), Linear.ForwardCore
(src/Idrak/Layers/Linear.cs:165), GEMM dispatch (src/Idrak.Gpu/Cuda/CudaBackend.cs:1306-1471).
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, scratch, stream_ptr

ACT_NONE, ACT_GELU, ACT_GELU_GRAD, ACT_GELU_D, ACT_MUL_AUX = 0, 1, 2, 3, 4
_ACT_IDS = {None: ACT_NONE, "none": ACT_NONE, "gelu": ACT_GELU, "gelu_grad": ACT_GELU_GRAD, "gelu_d": ACT_GELU_D,
            "mul_aux": ACT_MUL_AUX}
_TWO_OUTPUTS = (ACT_GELU, ACT_GELU_D)


def _gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def _gelu_tanh_grad(x: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def gemm_reference(a, b, *, a_mn=False, b_mn=False, bias=None, residual=None, act=None, aux=None,
                   out=None, beta=False, alpha=1.0, out_dtype=None):
    """Plain PyTorch statement of the kernel's contract (fp32 math)."""
    A = a.float().t() if a_mn else a.float()          # [M, K]
    Bt = b.float() if b_mn else b.float().t()         # [K, N]
    v = (A @ Bt) * alpha
    if bias is not None:
        v = v + bias.float()
    aux_out = None
    if _ACT_IDS[act] == ACT_GELU:
        aux_out = v.to(a.dtype)
        v = _gelu_tanh(aux_out.float())
    elif _ACT_IDS[act] == ACT_GELU_GRAD:
        v = v * _gelu_tanh_grad(aux.float())
    elif _ACT_IDS[act] == ACT_GELU_D:
        aux_out = _gelu_tanh_grad(v).to(a.dtype)
        v = _gelu_tanh(v)
    elif _ACT_IDS[act] == ACT_MUL_AUX:
        v = v * aux.float()
    if residual is not None:
        v = v + residual.float()
    dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is not None:
        if beta:
            v = v + out.float()
        out.copy_(v.to(dtype))
        res = out
    else:
        res = v.to(dtype)
    return (res, aux_out) if _ACT_IDS[act] in _TWO_OUTPUTS else res


def _tuned_splits(a, b, a_mn, b_mn, M, N, K, default, out) -> int:
    """The measured split-K factor for few-row products of this shape class (decode-sized work is where the built-in
    rule is least sure): read from the tuning cache, measured once with a cold L2 when tuning is on."""
    from ..runtime.tuning import size_class, tuner
    t = tuner()
    shape = (size_class(M), N, K, int(a_mn), int(b_mn))
    known = t.lookup("gemm.splits", shape)
    if known is not None:
        return int(known)
    if not t.enabled or torch.cuda.is_current_stream_capturing():
        return default
    kblocks = (K + 63) // 64
    options = sorted({default, 1, 2, 4, 8} & set(range(1, kblocks + 1)) | {default})
    scratch_out = torch.empty_like(out)
    cands = {str(s): (lambda s=s: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=scratch_out, splits=s)) for s in options}
    return int(t.choose("gemm.splits", shape, cands, default=str(default), cold_l2=True))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: torch.Tensor | None = None, residual: torch.Tensor | None = None, act: str | None = None,
         aux: torch.Tensor | None = None, out: torch.Tensor | None = None, beta: bool = False,
         alpha: float = 1.0, out_dtype: torch.dtype | None = None, splits: int | None = None):
    """``C = epilogue(alpha * op(A) @ op(B))``.

    ``a``: ``[M, K]`` (``a_mn=False``) or stored ``[K, M]`` (``a_mn=True``).
    ``b``: ``[N, K]`` (``b_mn=False``, the ``nn.Linear`` weight layout) or stored ``[K, N]`` (``b_mn=True``).
    ``act='gelu'`` returns ``(C, pre_activation)``; ``act='gelu_grad'`` multiplies by ``gelu'(aux)``.
    ``act='gelu_d'`` returns ``(C, gelu'(pre_activation))`` - the derivative taken where the tanh is at hand - and
    ``act='mul_aux'`` multiplies by ``aux``: the pair a training step uses, its backward epilogue one multiply.
    ``beta=True`` accumulates into ``out``. ``splits=None`` lets the library choose a split-K factor.
    """
    if not a.is_cuda:
        return gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=residual, act=act, aux=aux,
                              out=out, beta=beta, alpha=alpha, out_dtype=out_dtype)
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16), (a.dtype, b.dtype)
    assert a.dim() == 2 and b.dim() == 2
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    K, M = (a.shape if a_mn else (a.shape[1], a.shape[0]))
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    lib = _native.lib()
    act_id = _ACT_IDS[act]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        assert not beta
    assert out.stride(1) == 1 and out.shape == (M, N)
    c_fp32 = 1 if out.dtype == torch.float32 else 0
    assert c_fp32 or out.dtype == torch.bfloat16
    aux_t = aux
    if act_id in _TWO_OUTPUTS and aux_t is None:
        aux_t = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    bn = 128 if N <= 128 else 256
    if splits is None:
        splits = lib.idrak_gemm_pick_splits(M, N, K, bn)
        if M <= 256 and not (beta or act_id):
            splits = _tuned_splits(a, b, a_mn, b_mn, M, N, K, splits, out)
    ws = None
    if splits > 1:
        ws = scratch("gemm_splitk", splits * M * N, torch.float32, a.device)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    rc = lib.idrak_gemm_bf16(
        a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
        out.data_ptr(), out.stride(0), c_fp32, M, N, K,
        ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0,
        act_id, ptr(aux_t), aux_t.stride(0) if aux_t is not None else 0,
        int(beta), float(alpha), int(splits), ptr(ws), 1 if a.dtype == torch.float16 else 0, stream_ptr())
    _native.check(rc, "idrak_gemm_bf16")
    return (out, aux_t) if act_id in _TWO_OUTPUTS else out


def weight_grad(dy2: torch.Tensor, x2: torch.Tensor, param: torch.Tensor | None):
    """dW = dy^T x for an ``nn.Linear``-layout weight. Written straight into ``param.grad`` (and ``None``
    returned) when the parameter takes direct gradient writes, else returned as a new tensor."""
    from . import _grad
    tgt = _grad.target(param)
    if tgt is None:
        return gemm(dy2, x2, a_mn=True, b_mn=True)
    g, accumulate = tgt
    gemm(dy2, x2, a_mn=True, b_mn=True, out=g, beta=accumulate)
    _grad.written(param)
    return None


def bias_grad(dy2: torch.Tensor, param: torch.Tensor | None, dy: torch.Tensor | None = None):
    """db = column sums of dy. ``dy`` is the gradient tensor as autograd delivered it: when the kernel that produced
    it left its column sums on it (``_idrak_colsum``, see ``rowops.norm_backward``) no pass over dy is made."""
    from . import _grad
    from .rowops import colsum
    ready = None
    tagged = getattr(dy, "_idrak_colsum", None) if dy is not None else None
    if tagged is not None and tagged[1] == dy._version and tagged[0].numel() == dy2.shape[1]:
        ready = tagged[0]
    tgt = _grad.target(param)
    if tgt is None:
        return colsum(dy2) if ready is None else ready.to(dy2.dtype)
    g, accumulate = tgt
    if ready is None:
        colsum(dy2, out=g, accumulate=accumulate)
    elif accumulate:
        g.add_(ready.to(g.dtype))
    else:
        g.copy_(ready)
    _grad.written(param)
    return None


class _Linear(torch.autograd.Function):
    """y = x @ W^T (+ b) (+ residual); W is [out, in] as in ``nn.Linear``."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        y = gemm(x2, weight, bias=bias, residual=r2)
        ctx.save_for_backward(x2, weight)
        ctx.params = (weight, bias)          # the Parameter objects, for direct gradient writes
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        return y.reshape(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import _grad
        from .rowops import colsum
        x2, weight = ctx.saved_tensors
        w_param, b_param = ctx.params
        dy2 = dy.reshape(-1, weight.shape[0])
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).reshape(*dy.shape[:-1], weight.shape[1])
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, x2, w_param)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = bias_grad(dy2, b_param, dy)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    if not x.is_cuda:
        y = torch.nn.functional.linear(x, weight, bias)
        return y + residual if residual is not None else y
    return _Linear.apply(x, weight, bias, residual)


# --------------------------------------------------------------------------- product with a low-rank term
def gemm_lowrank_reference(a, b, a2, b2, *, b_mn=False, bias=None, residual=None):
    """fp32 statement of ``gemm_lowrank``."""
    v = a.float() @ (b.float() if b_mn else b.float().t()) + a2.float() @ (b2.float() if b_mn else b2.float().t())
    if bias is not None:
        v = v + bias.float()
    if residual is not None:
        v = v + residual.float()
    return v.to(a.dtype)


def lowrank_supported(a: torch.Tensor, rank: int) -> bool:
    """Whether the fused kernel takes this product: bf16 on the device, rank a multiple of 8 up to 256."""
    return a.is_cuda and a.dtype == torch.bfloat16 and 0 < rank <= 256 and rank % 8 == 0 and a.shape[-1] % 8 == 0


def gemm_lowrank(a, b, a2, b2, *, b_mn: bool = False, bias=None, residual=None):
    """``C = A op(B) + A2 op(B2) (+ bias) (+ residual)`` in one kernel: the second pair is contracted after the first
    into the same accumulator. ``a`` ``[M, K]``, ``a2`` ``[M, R]``; ``b`` / ``b2`` are ``[N, K]`` / ``[N, R]`` or, with
    ``b_mn``, stored ``[K, N]`` / ``[R, N]``."""
    if not lowrank_supported(a, a2.shape[1]):
        return gemm_lowrank_reference(a, b, a2, b2, b_mn=b_mn, bias=bias, residual=residual)
    a, b, a2, b2 = (t if t.stride(-1) == 1 else t.contiguous() for t in (a, b, a2, b2))
    M, K = a.shape
    R = a2.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == K and a2.shape[0] == M
    assert tuple(b2.shape) == ((R, N) if b_mn else (N, R)), (b2.shape, R, N)
    assert a.dtype == b.dtype == a2.dtype == b2.dtype == torch.bfloat16
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    rc = _native.lib().idrak_gemm_lowrank(
        a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), int(b_mn), a2.data_ptr(), a2.stride(0), b2.data_ptr(),
        b2.stride(0), out.data_ptr(), out.stride(0), M, N, K, R, ptr(bias), ptr(residual),
        residual.stride(0) if residual is not None else 0, stream_ptr())
    _native.check(rc, "idrak_gemm_lowrank")
    return out


class _LowRankLinear(torch.autograd.Function):
    """``y = x W^T + (x A^T) B^T (+ b) (+ residual)``. ``A`` ``[R, in]`` stacks the down matrices of the adapters on this
    projection and ``B`` ``[out, R]`` their scaled up matrices, each in its own column block and zero outside its slice
    of the output. Forward: one small product for ``x A^T`` and one product for the rest; backward likewise."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, A, B):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        t = gemm(x2, A)                                                       # [M, R]
        y = gemm_lowrank(x2, weight, t, B, bias=bias, residual=r2)
        ctx.save_for_backward(x2, weight, A, B, t)
        ctx.params = (weight, bias)
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return y.reshape(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, A, B, t = ctx.saved_tensors
        w_param, b_param = ctx.params
        dy2 = dy.reshape(-1, weight.shape[0])
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        dx = dw = db = dres = dA = dB = None
        dt = gemm(dy2, B, b_mn=True)                                          # [M, R]
        if ctx.needs_input_grad[0]:
            dx = gemm_lowrank(dy2, weight, dt, A, b_mn=True).reshape(*dy.shape[:-1], weight.shape[1])
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, x2, w_param)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = bias_grad(dy2, b_param, dy)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        if ctx.needs_input_grad[4]:
            dA = gemm(dt, x2, a_mn=True, b_mn=True)                           # [R, in]
        if ctx.needs_input_grad[5]:
            dB = gemm(dy2, t, a_mn=True, b_mn=True)                           # [out, R]
        return dx, dw, db, dres, dA, dB


def lowrank_linear(x, weight, bias, residual, A, B):
    """``x W^T + (x A^T) B^T (+ bias) (+ residual)`` with the low-rank term inside the base product's kernel."""
    if not lowrank_supported(x, A.shape[0]):
        y = torch.nn.functional.linear(x, weight, bias) + torch.nn.functional.linear(torch.nn.functional.linear(x, A), B)
        return y + residual if residual is not None else y
    return _LowRankLinear.apply(x, weight, bias, residual, A, B)
