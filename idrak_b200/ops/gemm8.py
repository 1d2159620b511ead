"""8-bit floating-point (e4m3) tensor-core products.

``quantize_rows(x)`` turns a bf16 matrix into e4m3 codes and one fp32 scale per row (``max|row| / 448``).
``gemm8(aq, a_scale, bq, b_scale)`` multiplies two such K-major operands - activations ``[M, K]`` and a weight in
``nn.Linear`` layout ``[N, K]`` - on the tcgen05 ``kind::f8f6f4`` path with fp32 accumulation and applies
``a_scale[m] * b_scale[n]`` (and an optional bias) in the epilogue; the result is bf16.
``linear_fp8(x, weight)`` does both for a forward product (the weight may be passed already quantised).

On CPU tensors the same functions run a plain PyTorch statement of the arithmetic (``torch.float8_e4m3fn`` for the
rounding), which is also what the GPU tests compare against.

Reference: Float8 products and their quantisers - gemm8_e4m3_f32, quant_rows_e4m3, quant_cols_e4m3
(src/Idrak.Gpu/Cuda/PtxKernels.EightBit.cs:17-23), Tensor.MatMul's Float8 branch and Float8Weight
(src/Idrak/Layers/Float8Weight.cs).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ._util import ptr, stream_ptr

E4M3_MAX = 448.0
_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    _native.bind("idrak_quant_rows_e4m3", i, [vp, i, vp, i, vp, i, i, vp])
    _native.bind("idrak_dequant_rows_e4m3", i, [vp, i, vp, vp, i, i, i, vp])
    _native.bind("idrak_gemm_fp8", i, [vp, i, vp, i, vp, i, i, i, i, vp, vp, vp, vp])
    _BOUND = True


@dataclass
class Float8Rows:
    """e4m3 codes ``[rows, K]`` (uint8 storage) with one fp32 scale per row."""
    codes: torch.Tensor
    scales: torch.Tensor

    @property
    def shape(self):
        return self.codes.shape

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return dequantize_rows(self, dtype)


def quantize_rows_reference(x: torch.Tensor) -> Float8Rows:
    xf = x.float()
    mx = xf.abs().amax(dim=1)
    scales = torch.where(mx > 0, mx / E4M3_MAX, torch.ones_like(mx))
    q = (xf / scales[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return Float8Rows(q.view(torch.uint8), scales)


def quantize_rows(x: torch.Tensor) -> Float8Rows:
    """Per-row symmetric quantisation of a 2-D bf16 matrix to e4m3."""
    assert x.dim() == 2
    if not (x.is_cuda and x.dtype == torch.bfloat16) or x.shape[1] % 8:
        return quantize_rows_reference(x)
    _bind()
    x = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 else x.contiguous()
    rows, K = x.shape
    codes = torch.empty((rows, K), dtype=torch.uint8, device=x.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _native.lib().idrak_quant_rows_e4m3(x.data_ptr(), x.stride(0), codes.data_ptr(), K, scales.data_ptr(), rows, K,
                                             stream_ptr())
    _native.check(rc, "idrak_quant_rows_e4m3")
    return Float8Rows(codes, scales)


def dequantize_rows(q: Float8Rows, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    codes, scales = q.codes, q.scales
    if not codes.is_cuda or dtype != torch.bfloat16 or codes.shape[1] % 2:
        return (codes.view(torch.float8_e4m3fn).float() * scales[:, None].float()).to(dtype)
    _bind()
    rows, K = codes.shape
    out = torch.empty((rows, K), dtype=torch.bfloat16, device=codes.device)
    rc = _native.lib().idrak_dequant_rows_e4m3(codes.data_ptr(), codes.stride(0), scales.data_ptr(), out.data_ptr(), K,
                                               rows, K, stream_ptr())
    _native.check(rc, "idrak_dequant_rows_e4m3")
    return out


def gemm8_reference(a: Float8Rows, b: Float8Rows, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 statement: (codes_a @ codes_b^T) * scale_a[m] * scale_b[n] (+ bias), rounded to bf16."""
    A = a.codes.view(torch.float8_e4m3fn).float()
    B = b.codes.view(torch.float8_e4m3fn).float()
    v = (A @ B.t()) * a.scales.float()[:, None] * b.scales.float()[None, :]
    if bias is not None:
        v = v + bias.float()
    return v.to(torch.bfloat16)


def gemm8(a: Float8Rows, b: Float8Rows, bias: Optional[torch.Tensor] = None,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C[M, N] = (A_codes @ B_codes^T) * a.scales[:, None] * b.scales[None, :] (+ bias)`` in bf16.
    ``a``: ``[M, K]``, ``b``: ``[N, K]`` (both K-major); K must be a multiple of 16."""
    M, K = a.codes.shape
    N, Kb = b.codes.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if not a.codes.is_cuda or K % 16:
        res = gemm8_reference(a, b, bias)
        if out is not None:
            out.copy_(res)
            return out
        return res
    _bind()
    ac = a.codes if a.codes.stride(1) == 1 and a.codes.stride(0) % 16 == 0 else a.codes.contiguous()
    bc = b.codes if b.codes.stride(1) == 1 and b.codes.stride(0) % 16 == 0 else b.codes.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=ac.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N
    rc = _native.lib().idrak_gemm_fp8(ac.data_ptr(), ac.stride(0), bc.data_ptr(), bc.stride(0), out.data_ptr(),
                                      out.stride(0), M, N, K, a.scales.data_ptr(), b.scales.data_ptr(), ptr(bias),
                                      stream_ptr())
    _native.check(rc, "idrak_gemm_fp8")
    return out


def linear_fp8(x: torch.Tensor, weight, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W^T + b`` with both operands rounded to e4m3 (per-row scales). ``weight`` is a bf16 ``[out, in]`` matrix or
    a ``Float8Rows`` made from one (quantise a frozen weight once and reuse it). Forward only."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    wq = weight if isinstance(weight, Float8Rows) else quantize_rows(weight.to(torch.bfloat16))
    y = gemm8(quantize_rows(x2.to(torch.bfloat16)), wq, bias)
    return y.reshape(*shape[:-1], wq.codes.shape[0])
