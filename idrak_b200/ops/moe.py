"""Routed experts on the device: top-k routing, permutation into per-expert segments, grouped tcgen05 products and the
weighted recombination, forward and backward, with no host read anywhere (a routed layer records into a CUDA graph).

``routed_experts(x, router, up, down, k, ...)`` takes the experts' weights stacked: ``up [E, (2) ff, dim]`` (gate rows then
up rows when gated), ``down [E, dim, ff]``. The plain PyTorch statement ``routed_experts_reference`` is the oracle and the
CPU path.

Data flow on the GPU (T tokens, A = T k assignments, rows = A + padding so every expert segment is whole 128-row tiles):

    logits = x router^T (fp32)            dense GEMM
    top_i, top_w, probs                   route_choose (ties: lowest expert id)
    plan (dst_of, row_of, tile_group ..)  route_count / route_offsets / route_place (stable, deterministic)
    xp   = x[row_of]                      route_gather
    gu   = xp  up_e^T                     grouped GEMM, expert per row tile
    h    = act(gate) * up                 gated activation kernel (or the plain activation)
    yp   = h down_e^T                     grouped GEMM
    out  = sum_k w yp[dst_of] (+res)      route_combine

Backward mirrors it: the weighted scatter of dy is a gather with weights, the input gradients are grouped products with
the weights read MN-major, the weight gradients are one grouped product per matrix in which expert e contracts over its own
rows only, and the router receives d(weights) through the softmax / top-k renormalisation.

Reference: MixtureOfExperts (src/Idrak/Layers/MixtureOfExperts.cs:34), routing kernels
(src/Idrak.Gpu/Cuda/PtxKernels.Routing.cs:12-35).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from ._util import ptr, stream_ptr
from .gemm import gemm
from .rowops import GATE_KINDS, _gate_ref


def _act_ref(h, kind):
    if kind == "gelu":
        return torch.nn.functional.gelu(h, approximate="tanh")
    if kind == "relu":
        return torch.relu(h)
    return torch.nn.functional.silu(h)


def route_reference(logits: torch.Tensor, k: int, normalize: bool):
    """softmax -> top-k with ties to the lowest expert id -> optional renormalisation. Returns (ids, weights, probs)."""
    probs = torch.softmax(logits.float(), -1)
    # stable descending sort: among equal probabilities the lower index comes first
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :k]
    w = probs.gather(1, order)
    if normalize:
        w = w / w.sum(-1, keepdim=True)
    return order.to(torch.int32), w, probs


def routed_experts_reference(x, router, up, down, k, normalize=True, gated=True, kind="silu", residual=None):
    """The loop over experts, in the dtype of ``x`` with fp32 routing and accumulation."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    ids, w, _ = route_reference(torch.nn.functional.linear(x2.float(), router.float()), k, normalize)
    out = torch.zeros_like(x2, dtype=torch.float32)
    E = up.shape[0]
    for e in range(E):
        rows, slot = torch.nonzero(ids == e, as_tuple=True)
        if rows.numel() == 0:
            continue
        h = torch.nn.functional.linear(x2[rows], up[e])
        if gated:
            ff = h.shape[-1] // 2
            h = _gate_ref(h[..., :ff], GATE_KINDS[kind]) * h[..., ff:]
        else:
            h = _act_ref(h, kind)
        y = torch.nn.functional.linear(h.to(x.dtype), down[e])
        out.index_add_(0, rows, y.float() * w[rows, slot][:, None])
    out = out.to(x.dtype).reshape(shape)
    return out + residual if residual is not None else out


class RoutePlan:
    """Device-side description of one routing: where every (token, pick) goes among the expert segments."""

    def __init__(self, top_i: torch.Tensor, experts: int):
        lib = _native.lib()
        T, k = top_i.shape
        A = T * k
        dev = top_i.device
        self.T, self.k, self.E = T, k, experts
        self.cap = lib.idrak_route_capacity(T, k, experts)
        blocks = lib.idrak_route_blocks(A)
        i32 = dict(dtype=torch.int32, device=dev)
        self.block_hist = torch.empty(blocks * experts, **i32)
        self.seg_start = torch.empty(experts, **i32)
        self.seg_count = torch.empty(experts, **i32)
        self.tile_group = torch.empty(self.cap // 128, **i32)
        self.group_kb = torch.empty(experts + 1, **i32)
        self.meta = torch.empty(4, **i32)
        self.dst_of = torch.empty(A, **i32)
        self.row_of = torch.empty(self.cap, **i32)
        rc = lib.idrak_route_plan(top_i.data_ptr(), A, experts, self.cap, self.block_hist.data_ptr(),
                                  self.seg_start.data_ptr(), self.seg_count.data_ptr(), self.tile_group.data_ptr(),
                                  self.group_kb.data_ptr(), self.meta.data_ptr(), self.dst_of.data_ptr(),
                                  self.row_of.data_ptr(), stream_ptr())
        _native.check(rc, "idrak_route_plan")

    def gather(self, src: torch.Tensor, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out[dst] = src[token of dst] (* weights[assignment])``; padding rows are zeros."""
        C = src.shape[-1]
        out = torch.empty((self.cap, C), dtype=src.dtype, device=src.device)
        rc = _native.lib().idrak_route_gather(src.data_ptr(), src.stride(0), self.row_of.data_ptr(), ptr(weights),
                                              self.meta.data_ptr(), self.k, C, self.cap, out.data_ptr(), stream_ptr())
        _native.check(rc, "idrak_route_gather")
        return out

    def combine(self, y: torch.Tensor, weights: Optional[torch.Tensor], residual: Optional[torch.Tensor] = None,
                grad: Optional[torch.Tensor] = None, want_out: bool = True):
        """``out[t] = sum_k weights[t, k] y[dst(t, k)] (+ residual[t])``; with ``grad`` also
        ``dw[t, k] = <grad[t], y[dst(t, k)]>``. Returns (out or None, dw or None)."""
        C = y.shape[-1]
        out = torch.empty((self.T, C), dtype=y.dtype, device=y.device) if want_out else None
        dw = torch.empty((self.T, self.k), dtype=torch.float32, device=y.device) if grad is not None else None
        rc = _native.lib().idrak_route_combine(y.data_ptr(), self.dst_of.data_ptr(), ptr(weights), ptr(residual),
                                               ptr(grad), ptr(dw), self.T, self.k, C, ptr(out), stream_ptr())
        _native.check(rc, "idrak_route_combine")
        return out, dw

    def rows_product(self, a: torch.Tensor, stacked: torch.Tensor, transpose_weights: bool) -> torch.Tensor:
        """``a[rows of e] @ stacked[e]^T`` (``transpose_weights=False``: stacked ``[E, N, K]``) or
        ``a[rows of e] @ stacked[e]`` (``True``: stacked ``[E, K, N]``)."""
        E = stacked.shape[0]
        K = a.shape[1]
        N = stacked.shape[2] if transpose_weights else stacked.shape[1]
        out = torch.empty((self.cap, N), dtype=a.dtype, device=a.device)
        rc = _native.lib().idrak_gemm_grouped_rows(a.data_ptr(), a.stride(0), stacked.data_ptr(), stacked.stride(1),
                                                   int(transpose_weights), out.data_ptr(), N, self.cap, N, K, E,
                                                   self.tile_group.data_ptr(), self.meta.data_ptr(), stream_ptr())
        _native.check(rc, "idrak_gemm_grouped_rows")
        return out

    def weight_grads(self, dy: torch.Tensor, x: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """``[E, M, N]`` with ``out[e] = dy[rows of e]^T @ x[rows of e]``."""
        M, N = dy.shape[1], x.shape[1]
        out = torch.empty((self.E, M, N), dtype=out_dtype, device=dy.device)
        rc = _native.lib().idrak_gemm_grouped_k(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), out.data_ptr(), N,
                                                int(out_dtype == torch.float32), 0, self.cap, M, N, self.E,
                                                self.group_kb.data_ptr(), stream_ptr())
        _native.check(rc, "idrak_gemm_grouped_k")
        return out


def route_choose(logits: torch.Tensor, k: int, normalize: bool):
    """Device top-k routing of fp32 ``logits [T, E]``: (ids int32 [T, k], weights fp32 [T, k], probs fp32 [T, E])."""
    T, E = logits.shape
    dev = logits.device
    top_i = torch.empty((T, k), dtype=torch.int32, device=dev)
    top_w = torch.empty((T, k), dtype=torch.float32, device=dev)
    probs = torch.empty((T, E), dtype=torch.float32, device=dev)
    rc = _native.lib().idrak_route_choose(logits.data_ptr(), T, E, k, int(normalize), top_i.data_ptr(), top_w.data_ptr(),
                                          probs.data_ptr(), stream_ptr())
    _native.check(rc, "idrak_route_choose")
    return top_i, top_w, probs


def _gated_forward(gu: torch.Tensor, kind_id: int) -> torch.Tensor:
    rows, two = gu.shape
    out = torch.empty((rows, two // 2), dtype=gu.dtype, device=gu.device)
    _native.check(_native.lib().idrak_gated_fwd(gu.data_ptr(), out.data_ptr(), rows, two // 2, kind_id, stream_ptr()),
                  "idrak_gated_fwd")
    return out


def _gated_backward(gu: torch.Tensor, dh: torch.Tensor, kind_id: int) -> torch.Tensor:
    rows, two = gu.shape
    dgu = torch.empty_like(gu)
    _native.check(_native.lib().idrak_gated_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), rows, two // 2, kind_id,
                                                stream_ptr()), "idrak_gated_bwd")
    return dgu


class _RoutedExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, router, up, down, residual, k, normalize, gated, kind):
        T, dim = x2.shape
        E = up.shape[0]
        logits = gemm(x2, router, out_dtype=torch.float32)
        top_i, top_w, probs = route_choose(logits, k, normalize)
        plan = RoutePlan(top_i, E)
        xp = plan.gather(x2)
        gu = plan.rows_product(xp, up, False)
        if gated:
            h = _gated_forward(gu, GATE_KINDS[kind])
        else:
            h = _act_ref(gu.float(), kind).to(gu.dtype)
        yp = plan.rows_product(h, down, False)
        out, _ = plan.combine(yp, top_w, residual)
        ctx.plan, ctx.cfg = plan, (k, normalize, gated, kind, residual is not None)
        ctx.save_for_backward(x2, router, up, down, xp, gu, h, yp, top_i, top_w, probs)
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, router, up, down, xp, gu, h, yp, top_i, top_w, probs = ctx.saved_tensors
        plan = ctx.plan
        k, normalize, gated, kind, has_res = ctx.cfg
        dy = dy.contiguous()
        # d(weights): what each pick's output contributed
        _, dw = plan.combine(yp, None, None, grad=dy, want_out=False)
        dyp = plan.gather(dy, top_w.reshape(-1))                       # rows of dy scaled by the pick's weight
        d_down = plan.weight_grads(dyp, h)                             # [E, dim, ff]
        dh = plan.rows_product(dyp, down, True)                        # [cap, ff]
        if gated:
            dgu = _gated_backward(gu, dh, GATE_KINDS[kind])
        else:
            g = gu.float().requires_grad_()
            with torch.enable_grad():
                a = _act_ref(g, kind)
            dgu = torch.autograd.grad(a, g, dh.float())[0].to(gu.dtype)
        d_up = plan.weight_grads(dgu, xp)                              # [E, (2) ff, dim]
        dxp = plan.rows_product(dgu, up, True)                         # [cap, dim]
        dx, _ = plan.combine(dxp, None)
        # router: weights -> (renormalised) top-k probabilities -> softmax
        picked = probs.gather(1, top_i.long())
        if normalize:
            s = picked.sum(-1, keepdim=True)
            dpicked = (dw - (dw * top_w).sum(-1, keepdim=True)) / s
        else:
            dpicked = dw
        dprobs = torch.zeros_like(probs).scatter_(1, top_i.long(), dpicked)
        dlogits = probs * (dprobs - (probs * dprobs).sum(-1, keepdim=True))
        dl16 = dlogits.to(x2.dtype)
        dx = dx + gemm(dl16, router, b_mn=True)
        d_router = gemm(dl16, x2, a_mn=True, b_mn=True)
        return dx, d_router, d_up, d_down, (dy if has_res else None), None, None, None, None


def supported(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor, gated: bool, kind: str) -> bool:
    """Whether the device path takes these shapes: bf16 on CUDA, contraction sizes in whole 64-element blocks, weight
    gradient outputs in whole 128-row tiles, a multiple of 8 experts (the router product's output rows), a gate the
    activation kernel knows."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16):
        return False
    E, rows_up, dim = up.shape
    ff = down.shape[2]
    if E > 256 or E % 8 or dim % 128 or ff % 64 or rows_up % 128 or (gated and kind not in GATE_KINDS):
        return False
    return up.is_contiguous() and down.is_contiguous()


def routed_experts(x: torch.Tensor, router: torch.Tensor, up: torch.Tensor, down: torch.Tensor, k: int,
                   normalize: bool = True, gated: bool = True, kind: str = "silu",
                   residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sum_k w_k expert_{e_k}(x) (+ residual)`` with the top-k experts of ``softmax(x router^T)`` per token."""
    if not supported(x, up, down, gated, kind):
        return routed_experts_reference(x, router, up, down, k, normalize, gated, kind, residual)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    r2 = residual.reshape(-1, shape[-1]).contiguous() if residual is not None else None
    out = _RoutedExperts.apply(x2, router.to(x.dtype), up, down, r2, k, normalize, gated, kind)
    return out.reshape(shape)
