"""Layer-level fused autograd functions used by the decoder on the GPU.

``qkv_attention``  packed QKV buffer -> (RoPE in place) -> flash attention; the backward pass writes
                   dQ, dK, dV straight into one d(QKV) buffer (strided outputs) and un-rotates in place.
``mlp_gelu``       x -> GELU(x W1^T + b1) W2^T + b2 (+ residual) with the GELU and its derivative (one tanh for
                   both) inside the first GEMM's epilogue and the multiplication by that derivative inside the
                   epilogue of the backward GEMM
                   (the reference's gemm_tc_nn_gelu / gemm_tc_nt_gelugrad pair,
                   src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:80-144).
``mlp_gated``      x -> act(x Wg^T) * (x Wu^T) -> W2 (+ residual) with gate and up in one GEMM.

CPU tensors take the plain PyTorch statement of the same math.
"""
from __future__ import annotations

import math

import torch

from . import rowops
from .attention import attention_reference, flash_backward, flash_forward
from .gemm import bias_grad, gemm, weight_grad
from .rowops import GATE_KINDS, _gate_ref, colsum, rope_, rope_reference


def _split_qkv(qkv, H, Hkv, D):
    B, S, _ = qkv.shape
    q = qkv[..., : H * D].unflatten(-1, (H, D))
    k = qkv[..., H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
    return q, k, v


class _QkvAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, Hkv, D, causal, scale, rope_theta, rope_dim, rope_scale, positions, window=None,
                row_start=None, softcap=None):
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, H, Hkv, D)
        if rope_theta is not None:
            # the projection output is ours to overwrite: rotate q and k where they lie
            for t, heads in ((q, H), (k, Hkv)):
                rope_(t.flatten(0, 1), positions, rope_theta, rope_dim, rope_scale, False)
        out, lse = flash_forward(q, k, v, causal, scale, window, row_start, softcap)
        ctx.save_for_backward(qkv, out, lse, positions)
        ctx.cfg = (H, Hkv, D, causal, scale, rope_theta, rope_dim, rope_scale)
        ctx.modes = (window, row_start, softcap)
        # qkv was rotated through its raw pointer; its producer (a projection) does not need it again
        return out.reshape(B, S, H * D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, positions = ctx.saved_tensors
        H, Hkv, D, causal, scale, rope_theta, rope_dim, rope_scale = ctx.cfg
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, H, Hkv, D)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split_qkv(dqkv, H, Hkv, D)
        window, row_start, softcap = ctx.modes
        flash_backward(dout.reshape(B, S, H, D), q, k, v, out, lse, causal, scale, (dq, dk, dv), window, row_start,
                       softcap)
        if rope_theta is not None:
            for t in (dq, dk):
                rope_(t.flatten(0, 1), positions, rope_theta, rope_dim, rope_scale, True)
        return (dqkv,) + (None,) * 12


def qkv_attention(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int, causal: bool = True,
                  scale: float | None = None, rope_theta: float | None = None, rope_dim: int | None = None,
                  rope_scale: float = 1.0, positions: torch.Tensor | None = None, window: int | None = None,
                  row_start: torch.Tensor | None = None, softcap: float | None = None) -> torch.Tensor:
    """Self-attention over a packed ``[B, S, (H + 2*Hkv) * D]`` projection; returns ``[B, S, H*D]``.

    On the GPU the buffer is rotated in place (it must be a fresh projection output). ``window``, ``row_start``
    (``[B, S]`` first visible key per position: sequences packed into one row) and ``softcap`` as in
    ``ops.attention``."""
    B, S, _ = qkv.shape
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim in (64, 128):
        if positions is None and rope_theta is not None:
            positions = (torch.arange(S, device=qkv.device, dtype=torch.int32).repeat(B))
        return _QkvAttention.apply(qkv, heads, kv_heads, head_dim, causal, scale, rope_theta, rope_dim,
                                   rope_scale, positions, window, row_start, softcap)
    q, k, v = _split_qkv(qkv, heads, kv_heads, head_dim)
    if rope_theta is not None:
        pos = positions if positions is not None else torch.arange(S, device=qkv.device).repeat(B)
        q = rope_reference(q.reshape(B * S, heads, head_dim), pos, rope_theta, rope_dim, rope_scale).reshape(q.shape)
        k = rope_reference(k.reshape(B * S, kv_heads, head_dim), pos, rope_theta, rope_dim, rope_scale).reshape(k.shape)
    return attention_reference(q, k, v, causal, scale, window, row_start, softcap).reshape(B, S, heads * head_dim)


class _MlpGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
        h, dact = gemm(x2, w1, bias=b1, act="gelu_d")          # dact = gelu'(pre-activation), saved instead of it
        y = gemm(h, w2, bias=b2, residual=r2)
        ctx.save_for_backward(x2, w1, w2, dact, h)
        ctx.params = (w1, b1, w2, b2)
        ctx.flags = (b1 is not None, b2 is not None, residual is not None)
        return y.reshape(*shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, dact, h = ctx.saved_tensors
        has_b1, has_b2, has_res = ctx.flags
        dy2 = dy.reshape(-1, w2.shape[0])
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        p_w1, p_b1, p_w2, p_b2 = ctx.params
        dw2 = weight_grad(dy2, h, p_w2)
        db2 = bias_grad(dy2, p_b2, dy) if has_b2 else None
        dpre = gemm(dy2, w2, b_mn=True, act="mul_aux", aux=dact)
        dw1 = weight_grad(dpre, x2, p_w1)
        db1 = bias_grad(dpre, p_b1) if has_b1 else None
        dx = gemm(dpre, w1, b_mn=True).reshape(*dy.shape[:-1], w1.shape[1])
        return dx, dw1, db1, dw2, db2, (dy if has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    """``GELU(x W1^T + b1) W2^T + b2 (+ residual)``; weights in ``nn.Linear`` layout."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _MlpGelu.apply(x, w1, b1, w2, b2, residual)
    h = torch.nn.functional.gelu(torch.nn.functional.linear(x, w1, b1), approximate="tanh")
    y = torch.nn.functional.linear(h, w2, b2)
    return y + residual if residual is not None else y


class _MlpGated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wgu, bgu, w2, b2, residual, kind):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
        gu = gemm(x2, wgu, bias=bgu)
        Hd = gu.shape[1] // 2
        act = torch.empty((gu.shape[0], Hd), dtype=gu.dtype, device=gu.device)
        from .. import _native
        from ._util import stream_ptr
        _native.check(_native.lib().idrak_gated_fwd(gu.data_ptr(), act.data_ptr(), gu.shape[0], Hd, kind,
                                                    stream_ptr()), "gated_fwd")
        y = gemm(act, w2, bias=b2, residual=r2)
        ctx.save_for_backward(x2, wgu, w2, gu, act)
        ctx.params = (wgu, bgu, w2, b2)
        ctx.flags = (bgu is not None, b2 is not None, residual is not None, kind)
        return y.reshape(*shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .. import _native
        from ._util import stream_ptr
        x2, wgu, w2, gu, act = ctx.saved_tensors
        has_bgu, has_b2, has_res, kind = ctx.flags
        dy2 = dy.reshape(-1, w2.shape[0])
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        p_wgu, p_bgu, p_w2, p_b2 = ctx.params
        dw2 = weight_grad(dy2, act, p_w2)
        db2 = bias_grad(dy2, p_b2, dy) if has_b2 else None
        dact = gemm(dy2, w2, b_mn=True)
        dgu = torch.empty_like(gu)
        Hd = gu.shape[1] // 2
        _native.check(_native.lib().idrak_gated_bwd(gu.data_ptr(), dact.data_ptr(), dgu.data_ptr(), gu.shape[0], Hd,
                                                    kind, stream_ptr()), "gated_bwd")
        dwgu = weight_grad(dgu, x2, p_wgu)
        dbgu = bias_grad(dgu, p_bgu) if has_bgu else None
        dx = gemm(dgu, wgu, b_mn=True).reshape(*dy.shape[:-1], wgu.shape[1])
        return dx, dwgu, dbgu, dw2, db2, (dy if has_res else None), None


def mlp_gated(x, w_gate_up, b_gate_up, w_down, b_down, residual=None, kind: str = "silu"):
    """``down(act(gate(x)) * up(x)) (+ residual)`` with ``w_gate_up = [gate; up]`` stacked on the output dim."""
    k = GATE_KINDS[kind]
    if x.is_cuda and x.dtype == torch.bfloat16 and (w_gate_up.shape[0] // 2) % 8 == 0:
        return _MlpGated.apply(x, w_gate_up, b_gate_up, w_down, b_down, residual, k)
    gu = torch.nn.functional.linear(x, w_gate_up, b_gate_up)
    Hd = gu.shape[-1] // 2
    y = torch.nn.functional.linear(_gate_ref(gu[..., :Hd], k) * gu[..., Hd:], w_down, b_down)
    return y + residual if residual is not None else y
