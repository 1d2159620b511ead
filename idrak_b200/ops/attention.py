"""Flash attention (training / prefill) on the tcgen05 kernels, with a plain PyTorch reference.

Tensors are ``[batch, seq, heads, head_dim]`` views; the last dim must be contiguous and the head dim
stride must equal ``head_dim`` (heads packed inside a row), which is what a fused QKV projection
produces — so q, k, v may be slices of one ``[B, S, 3*H*D]`` buffer and no copy is made.

Reference: Tensor.CausalAttention (src/Idrak.Abstraction/Tensors/Tensor.Decoding.cs:132),
flash_tc_{fwd,bwd_q,bwd_kv,delta} (src/Idrak.Gpu/Cuda/PtxKernels.FlashTensorCore.cs).
"""
from __future__ import annotations

import math

import torch

from .. import _native
from ._util import ptr, stream_ptr


def row_starts_from_spans(spans, batch: int, seq: int, device=None) -> torch.Tensor:
    """``[batch, seq]`` int32: for every position the first position of the sequence it belongs to, for sequences
    packed back to back as ``[(lo, hi), ...]`` in each row of the batch (positions outside every span start at
    themselves). This is what the attention kernels take as ``row_start``."""
    starts = torch.arange(seq, dtype=torch.int32)
    for lo, hi in spans:
        starts[lo:hi] = lo
    starts = starts[None, :].expand(batch, seq).contiguous()
    return starts.to(device) if device is not None else starts


def attention_reference(q, k, v, causal=True, scale=None, window=None, row_start=None, softcap=None):
    """fp32 softmax(QK^T)V with grouped heads. q: [B,Sq,H,D], k/v: [B,Skv,Hkv,D].

    ``window``: a query sees the ``window`` most recent keys only. ``row_start`` ``[B, Sq]``: the first key each
    query may see. ``softcap``: scores become ``softcap * tanh(score / softcap)``."""
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap:
        s = torch.tanh(s / softcap) * softcap
    if causal:
        off = Skv - Sq
        i = torch.arange(Sq, device=q.device)[:, None]
        j = torch.arange(Skv, device=q.device)[None, :]
        mask = j > i + off
        if window:
            mask = mask | (j <= i + off - window)
        s = s.masked_fill(mask, float("-inf"))
        if row_start is not None:
            below = j[None] < row_start.to(q.device).reshape(B, Sq, 1)
            s = s.masked_fill(below[:, None], float("-inf"))
    else:
        assert not window and row_start is None, "window and row_start need causal attention"
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def _check_layout(t: torch.Tensor, name: str):
    B, S, H, D = t.shape
    assert t.dtype == torch.bfloat16, f"{name}: bf16 required"
    assert t.stride(3) == 1 and t.stride(2) == D, f"{name}: heads must be packed [H, D] inside a row"
    assert t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0, f"{name}: alignment"


def _row_start_arg(row_start, B, Sq, device):
    if row_start is None:
        return None
    rs = row_start.to(device=device, dtype=torch.int32).reshape(B, Sq).contiguous()
    return rs


def flash_forward(q, k, v, causal=True, scale=None, window=None, row_start=None, softcap=None):
    """Returns (out [B,Sq,H,D] contiguous, lse [B,H,Sq] fp32). ``window`` / ``row_start`` / ``softcap`` as in
    ``attention_reference``; ``row_start`` must not decrease along a row of the batch."""
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_layout(t, n)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    rs = _row_start_arg(row_start, B, Sq, q.device)
    rc = _native.lib().idrak_flash_fwd_ex(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, H, Hkv, Sq, Skv, D,
        q.stride(1), k.stride(1), v.stride(1), H * D, q.stride(0), k.stride(0), v.stride(0),
        float(scale), int(causal), int(window or 0), ptr(rs), float(softcap or 0.0), stream_ptr())
    _native.check(rc, "idrak_flash_fwd_ex")
    return out, lse


def flash_backward(dout, q, k, v, out, lse, causal=True, scale=None, grads=None, window=None, row_start=None,
                   softcap=None):
    """Returns (dq, dk, dv) shaped like q, k, v. ``grads`` may supply the three output views (rows holding
    heads packed [heads, D], any row stride, batch stride = rows * row stride), e.g. slices of one d(QKV)."""
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    lib = _native.lib()
    dout = dout.contiguous()
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    if grads is None:
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Skv, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Skv, Hkv, D), dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = grads
        for g, rows in ((dq, Sq), (dk, Skv), (dv, Skv)):
            assert g.stride(3) == 1 and g.stride(2) == D and g.stride(0) == rows * g.stride(1)
    rs = _row_start_arg(row_start, B, Sq, q.device)
    rc = lib.idrak_flash_bwd_ex(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
        delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, Hkv, Sq, Skv, D,
        q.stride(1), k.stride(1), v.stride(1), q.stride(0), k.stride(0), v.stride(0),
        dq.stride(1), dk.stride(1), dv.stride(1), float(scale), int(causal), int(window or 0), ptr(rs),
        float(softcap or 0.0), stream_ptr())
    _native.check(rc, "idrak_flash_bwd_ex")
    return dq, dk, dv


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, window, row_start, softcap):
        out, lse = flash_forward(q, k, v, causal, scale, window, row_start, softcap)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (causal, scale, window, row_start, softcap)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        causal, scale, window, row_start, softcap = ctx.cfg
        dq, dk, dv = flash_backward(dout, q, k, v, out, lse, causal, scale, None, window, row_start, softcap)
        return dq, dk, dv, None, None, None, None, None


def attention(q, k, v, causal: bool = True, scale: float | None = None, window: int | None = None,
              row_start: torch.Tensor | None = None, softcap: float | None = None) -> torch.Tensor:
    """Scaled dot-product attention; q [B,Sq,H,D], k/v [B,Skv,Hkv,D]; returns [B,Sq,H,D].

    Optional modes (sliding ``window``, per-row first key ``row_start`` for packed sequences, tanh ``softcap``)
    run inside the same kernels, forward and backward."""
    D = q.shape[-1]
    modes = bool(window) or row_start is not None or bool(softcap)
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        return _FlashAttention.apply(q, k, v, causal, scale, window, row_start, softcap)
    if q.is_cuda:
        raise NotImplementedError(f"attention on CUDA needs bf16 and head_dim 64 or 128 (got {q.dtype}, {D})")
    if modes:
        return attention_reference(q, k, v, causal, scale, window, row_start, softcap)
    if q.shape[1] == k.shape[1]:
        # host path: the library's fused attention (the explicit statement above stays the oracle of the tests)
        H, Hkv = q.shape[2], k.shape[2]
        kk, vv = (k, v) if H == Hkv else (k.repeat_interleave(H // Hkv, dim=2), v.repeat_interleave(H // Hkv, dim=2))
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                             is_causal=causal, scale=scale)
        return o.transpose(1, 2)
    return attention_reference(q, k, v, causal, scale)
