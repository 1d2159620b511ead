"""Serving-side ops: paged KV cache writes, decode attention over block tables, device-side sampling.

Each op runs the sm_100a kernel on CUDA tensors and a plain PyTorch statement of the same math on CPU
tensors (the oracle of the GPU tests and the engine's CPU path).

Reference: Tensor.AttentionRows / KeyValueWrite / SampleRows (src/Idrak.Abstraction/Tensors/Tensor.Decoding.cs),
KeyValueCache (src/Idrak.Abstraction/Generation/Decoding.cs:243), TokenSampler (TokenSamplers.cs).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native
from ._util import ptr, scratch, stream_ptr

_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, f, ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
    _native.bind("idrak_decode_partial_floats", ll, [i, i, i, i])
    _native.bind("idrak_paged_decode", i, [vp, C.c_longlong, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, i, vp])
    _native.bind("idrak_paged_decode_kv", i, [vp, C.c_longlong, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, i, vp])
    _native.bind("idrak_norm_rope_kv", i, [vp, ll, vp, vp, vp, vp, vp, vp, vp, vp, f, f, f, i, i, i, i, i, i, vp])
    _native.bind("idrak_kv_write_paged", i, [vp, vp, ll, vp, vp, vp, i, i, vp])
    _native.bind("idrak_argmax_rows", i, [vp, i, i, i, ll, vp, vp])
    _native.bind("idrak_sample_rows", i, [vp, i, i, i, ll, vp, vp, vp, vp, vp, vp, vp, i, vp, vp, vp, vp, C.c_uint, vp])
    _BOUND = True


# --------------------------------------------------------------------------- KV cache
def kv_write_paged(k_src: torch.Tensor, v_src: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor) -> None:
    """Write the new tokens' keys / values (``[tokens, Hkv, D]`` views with packed heads) into cache slots
    ``slots[t] = block * block_size + offset`` (negative = skip)."""
    tokens, Hkv, D = k_src.shape
    row = Hkv * D
    if not k_src.is_cuda:
        flat_k, flat_v = k_cache.view(-1, row), v_cache.view(-1, row)
        keep = slots >= 0
        flat_k[slots[keep].long()] = k_src.reshape(tokens, row)[keep]
        flat_v[slots[keep].long()] = v_src.reshape(tokens, row)[keep]
        return
    _bind()
    assert k_src.stride(2) == 1 and k_src.stride(1) == D and v_src.stride(0) == k_src.stride(0)
    assert slots.dtype == torch.int32
    rc = _native.lib().idrak_kv_write_paged(k_src.data_ptr(), v_src.data_ptr(), k_src.stride(0), slots.data_ptr(),
                                            k_cache.data_ptr(), v_cache.data_ptr(), tokens, row, stream_ptr())
    _native.check(rc, "idrak_kv_write_paged")


def quantize_kv_reference(x: torch.Tensor):
    """int8 codes and one fp32 scale per (token, head) of ``[tokens, heads, D]``: scale = max|x| / 127."""
    xf = x.float()
    mx = xf.abs().amax(-1)
    scale = torch.where(mx > 0, mx / 127.0, torch.ones_like(mx))
    q = torch.round(xf / scale[..., None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def norm_rope_kv(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int, positions: Optional[torch.Tensor],
                 slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                 k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
                 q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                 eps: float = 1e-6, theta: Optional[float] = None, rot_dim: Optional[int] = None,
                 freq_scale: float = 1.0) -> None:
    """In place on the packed projection ``[T, (H + 2 Hkv) D]``: per-head RMS norm of queries and keys (when weights
    are given), RoPE of both (when ``theta`` is given), and the write of keys / values into the paged cache rows
    ``slots`` - bf16, or int8 codes with one scale per (slot, kv head) when ``k_scale`` / ``v_scale`` are given. One
    kernel launch on the GPU; the CPU path composes the same steps."""
    T = qkv.shape[0]
    H, Hkv, D = heads, kv_heads, head_dim
    rot = (rot_dim or D) if theta is not None else 0
    fused = (qkv.is_cuda and qkv.dtype == torch.bfloat16 and D in (64, 128, 256) and rot % 64 == 0
             and qkv.stride(1) == 1)
    if fused:
        _bind()
        int8 = k_scale is not None
        rc = _native.lib().idrak_norm_rope_kv(
            qkv.data_ptr(), qkv.stride(0), ptr(positions), ptr(slots), ptr(k_cache), ptr(v_cache), ptr(k_scale),
            ptr(v_scale), ptr(q_norm_weight), ptr(k_norm_weight), float(eps), float(theta or 10000.0), float(freq_scale),
            int(rot), T, H, Hkv, D, int(int8), stream_ptr())
        _native.check(rc, "idrak_norm_rope_kv")
        return
    from .rowops import rope_
    qk = qkv[:, : (H + Hkv) * D].unflatten(-1, (H + Hkv, D))

    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    if q_norm_weight is not None:
        qk[:, :H].copy_(rms(qk[:, :H], q_norm_weight))
    if k_norm_weight is not None:
        qk[:, H:].copy_(rms(qk[:, H:], k_norm_weight))
    if theta is not None:
        rope_(qk, positions, theta, rot_dim, freq_scale)
    if slots is None:
        return
    k = qkv[:, H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[:, (H + Hkv) * D:].unflatten(-1, (Hkv, D))
    if k_scale is None:
        kv_write_paged(k, v, slots, k_cache, v_cache)
        return
    keep = slots >= 0
    idx = slots[keep].long()
    for src, cache, scales in ((k, k_cache, k_scale), (v, v_cache, v_scale)):
        q8, sc = quantize_kv_reference(src[keep])
        cache.view(-1, Hkv, D)[idx] = q8
        scales.view(-1, Hkv)[idx] = sc


def paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, scale=None, window: int = 0,
                           k_scale=None, v_scale=None):
    if k_scale is not None:
        k_cache = (k_cache.float() * k_scale.view(*k_cache.shape[:3], 1)).to(q.dtype)
        v_cache = (v_cache.float() * v_scale.view(*v_cache.shape[:3], 1)).to(q.dtype)
    seqs, H, D = q.shape
    _, bs, Hkv, _ = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    for s in range(seqs):
        n = int(seq_lens[s])
        if n == 0:
            continue
        blocks = block_table[s, : (n + bs - 1) // bs].long()
        k = k_cache[blocks].reshape(-1, Hkv, D)[:n].float()
        v = v_cache[blocks].reshape(-1, Hkv, D)[:n].float()
        if window and n > window:
            k, v = k[n - window:], v[n - window:]
        k = k.repeat_interleave(H // Hkv, dim=1)
        v = v.repeat_interleave(H // Hkv, dim=1)
        sc = torch.einsum("hd,nhd->hn", q[s].float(), k) * scale
        out[s] = torch.einsum("hn,nhd->hd", torch.softmax(sc, -1), v)
    return out.to(q.dtype)


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, scale: Optional[float] = None, window: int = 0,
                 splits: Optional[int] = None, max_len_hint: Optional[int] = None,
                 k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence against its cached keys / values. q: ``[seqs, H, D]``. With ``k_scale`` /
    ``v_scale`` (``[blocks, block_size, Hkv]`` fp32) the caches hold int8 codes."""
    if not q.is_cuda:
        return paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, scale, window, k_scale, v_scale)
    _bind()
    seqs, H, D = q.shape
    _, bs, Hkv, _ = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    lib = _native.lib()
    if splits is None:
        # fill the machine: sequences x kv heads CTAs may be few; long contexts split along the keys
        ctas = seqs * Hkv
        longest = max_len_hint if max_len_hint is not None else block_table.shape[1] * bs
        splits = max(1, min(lib.idrak_sm_count() * 2 // max(ctas, 1), (longest + 255) // 256, 32))
    out = torch.empty(seqs, H, D, dtype=q.dtype, device=q.device)
    part = None
    if splits > 1:
        part = scratch("decode_partial", lib.idrak_decode_partial_floats(seqs, H, D, splits), torch.float32, q.device)
    if q.stride(2) != 1 or q.stride(1) != D or q.stride(0) % 8 or q.data_ptr() % 16:
        q = q.contiguous()                     # heads must be packed; sequences may be a strided view
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    rc = lib.idrak_paged_decode_kv(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), ptr(k_scale),
                                   ptr(v_scale), block_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), ptr(part),
                                   seqs, H, Hkv, D, bs, block_table.shape[1], splits, float(scale), int(window),
                                   stream_ptr())
    _native.check(rc, "idrak_paged_decode_kv")
    return out


# --------------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor, vocab: Optional[int] = None) -> torch.Tensor:
    """Greedy token per row (lowest id among ties). logits: ``[rows, ld]`` bf16 or fp32."""
    rows, ld = logits.shape
    vocab = vocab or ld
    if not logits.is_cuda:
        return logits[:, :vocab].float().argmax(-1).to(torch.int32)
    _bind()
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
    rc = _native.lib().idrak_argmax_rows(logits.data_ptr(), int(logits.dtype == torch.float32), rows, vocab,
                                         logits.stride(0), ids.data_ptr(), stream_ptr())
    _native.check(rc, "idrak_argmax_rows")
    return ids


def sample_rows_reference(logits, vocab, temperature, top_k, top_p, min_p, uniforms):
    """Same filtering as the kernel; ``uniforms[row]`` in [0,1) picks along the kept, sorted candidates."""
    out = []
    for r in range(logits.shape[0]):
        v = logits[r, :vocab].float() / max(float(temperature[r]), 1e-6)
        k = int(top_k[r]) if int(top_k[r]) > 0 else 64
        k = min(k, 64, vocab)
        vals, idx = torch.sort(v, descending=True, stable=True)
        vals, idx = vals[:k], idx[:k]
        pr = torch.exp(vals - vals[0])
        keep = k
        if float(min_p[r]) > 0:
            keep = max(int((pr >= float(min_p[r]) * pr[0]).sum()), 1)
        if float(top_p[r]) < 1:
            cum = torch.cumsum(pr[:keep] / pr.sum(), 0)
            c = int((cum < float(top_p[r])).sum()) + 1
            keep = max(min(c, keep), 1)
        cum = torch.cumsum(pr[:keep], 0)
        u = float(uniforms[r]) * float(cum[-1])
        pick = int((cum <= u).sum())
        out.append(int(idx[min(pick, keep - 1)]))
    return torch.tensor(out, dtype=torch.int32)


def penalise_reference(logits, vocab, history, repeat_penalty=None, presence_penalty=None, frequency_penalty=None):
    """The kernel's penalties: tokens seen in ``history`` (-1 = empty) are divided / multiplied by the repeat
    penalty (positive / negative logits), then lose the presence penalty and count x the frequency penalty."""
    out = logits[:, :vocab].float().clone()
    for r in range(out.shape[0]):
        h = history[r][history[r] >= 0].long()
        if h.numel() == 0:
            continue
        ids, counts = torch.unique(h, return_counts=True)
        v = out[r, ids]
        rp = float(repeat_penalty[r]) if repeat_penalty is not None else 1.0
        if rp != 1.0:
            v = torch.where(v > 0, v / rp, v * rp)
        if presence_penalty is not None:
            v = v - float(presence_penalty[r])
        if frequency_penalty is not None:
            v = v - float(frequency_penalty[r]) * counts.float()
        out[r, ids] = v
    return out


def sample_rows(logits: torch.Tensor, vocab: int, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, min_p: torch.Tensor, seeds: torch.Tensor, step: int,
                history: Optional[torch.Tensor] = None, repeat_penalty: Optional[torch.Tensor] = None,
                presence_penalty: Optional[torch.Tensor] = None, frequency_penalty: Optional[torch.Tensor] = None,
                return_logprobs: bool = False):
    """Sample one token per row on the device. Per-row settings are tensors on the logits' device
    (float32 / int32; ``seeds`` int64)."""
    rows = logits.shape[0]
    if not logits.is_cuda:
        u = torch.empty(rows)
        for r in range(rows):      # one stream per row, so a row's draw does not depend on its batch neighbours
            g = torch.Generator().manual_seed((int(seeds[r]) * 1000003 + step) & 0x7FFFFFFFFFFFFFFF)
            u[r] = torch.rand(1, generator=g)[0]
        if history is not None:
            logits = penalise_reference(logits, vocab, history, repeat_penalty, presence_penalty, frequency_penalty)
        ids = sample_rows_reference(logits, vocab, temperature, top_k, top_p, min_p, u)
        return (ids, torch.zeros(rows)) if return_logprobs else ids
    _bind()
    ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lp = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_logprobs else None
    rc = _native.lib().idrak_sample_rows(
        logits.data_ptr(), int(logits.dtype == torch.float32), rows, vocab, logits.stride(0), ids.data_ptr(), ptr(lp),
        temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), ptr(history),
        history.shape[1] if history is not None else 0, ptr(repeat_penalty), ptr(presence_penalty),
        ptr(frequency_penalty), seeds.data_ptr(), int(step), stream_ptr())
    _native.check(rc, "idrak_sample_rows")
    return (ids, lp) if return_logprobs else ids
