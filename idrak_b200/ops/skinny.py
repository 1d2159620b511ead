"""Few-row projections for decoding (at most 64 token rows): one launch per projection with its epilogue inside.

``skinny_linear(x, w, ...)`` computes ``x @ w.T`` on the cluster split-K kernel (``csrc/skinny_gemm.cu``) and, in the
same launch, any of: a folded RMS norm of ``x`` (``norm_eps``: ``w`` must carry the norm weight in its columns, see
``fold_norm``), a bias, a residual add, and - with ``gate`` - the gated activation of a stacked ``[gate; up]`` matrix.
``skinny_reference`` is the fp32 statement of the same thing and the CPU path.

Reference: the fused few-row GEMV family (src/Idrak.Gpu/Cuda/PtxKernels.Quantized.cs:454-495).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from ._util import ptr, stream_ptr
from .rowops import GATE_KINDS, _gate_ref

MAX_ROWS = 64
_KINDS = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "relu": 2, "reglu": 2}


def fold_norm(weight: torch.Tensor, norm_weight: torch.Tensor) -> torch.Tensor:
    """``weight * norm_weight[None, :]``: the projection that, applied to ``x * rstd``, equals ``norm(x) @ weight.T``."""
    return (weight.float() * norm_weight.float()[None, :]).to(weight.dtype)


def skinny_reference(x, w, bias=None, residual=None, gate: Optional[str] = None, norm_eps: Optional[float] = None):
    xf = x.float()
    if norm_eps is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + norm_eps)
    y = xf @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if gate is not None:
        ff = y.shape[-1] // 2
        y = _gate_ref(y[..., :ff], GATE_KINDS[gate]) * y[..., ff:]
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def supported(x: torch.Tensor, w: torch.Tensor, gate: Optional[str] = None) -> bool:
    return (x.is_cuda and _native.has("idrak_skinny_gemm") and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[0] <= MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (gate is None or (gate in _KINDS and (w.shape[0] // 2) % 8 == 0)))


def skinny_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, gate: Optional[str] = None,
                  norm_eps: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [M <= 64, K]``, ``w [N, K]`` (or ``[2 ff, K]`` with ``gate``) -> ``[M, N]`` (``[M, ff]``)."""
    if not supported(x, w, gate):
        return skinny_reference(x, w, bias, residual, gate, norm_eps)
    M, K = x.shape
    N = w.shape[0] // 2 if gate is not None else w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = _native.lib().idrak_skinny_gemm(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K, ptr(bias),
        ptr(residual), residual.stride(0) if residual is not None else 0, _KINDS[gate] if gate is not None else -1,
        float(norm_eps) if norm_eps is not None else -1.0, stream_ptr())
    _native.check(rc, "idrak_skinny_gemm")
    return out


# Rows of the weight matrix from which the dense GEMM (with its own split-K choice) streams a few-row product faster than
# the cluster kernel; measured at 64 activation rows, K = 4096: 6144 rows 23.7 / 24.4 us (few-row / dense), 7168 rows
# 25.5 / 25.3, 16032 rows 46.1 / 40.2, 32064 rows 78.6 / 61.1, 128256 rows 266 / 192; the stacked gate / up matrix with
# the activation: 28672 rows 73.9 us against 56.3 + 3 us for the dense product and the activation kernel.
DENSE_FROM_ROWS = 12288


def few_row_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None, gate: Optional[str] = None,
                   norm_eps: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A decode-sized product on whichever of the two kernels measured faster for the weight's size: the few-row cluster
    kernel (fused epilogues, small and medium weights) or the dense GEMM followed, for a gated pair, by the activation
    kernel (wide weights). A folded norm (``norm_eps``) exists only in the few-row kernel."""
    if norm_eps is not None or w.shape[0] < DENSE_FROM_ROWS or not x.is_cuda:
        return skinny_linear(x, w, bias, residual, gate, norm_eps, out)
    from .gemm import gemm
    if gate is None:
        return gemm(x, w, bias=bias, residual=residual, out=out)
    from .rowops import gated_activation
    y = gated_activation(gemm(x, w, bias=bias), gate)
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def skinny8_reference(x, w8, bias=None, residual=None, gate: Optional[str] = None):
    """fp32 statement of ``skinny8_linear``; ``w8`` is an ``Int8Weight`` ([in, out]; gated: out = [gate | up])."""
    y = x.float() @ w8.dequantize().to(x.device)
    if bias is not None:
        y = y + bias.float()
    if gate is not None:
        g, u = y.chunk(2, -1)
        act = {"silu": torch.nn.functional.silu, "swiglu": torch.nn.functional.silu, "relu": torch.relu, "reglu": torch.relu,
               "gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
               "geglu": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[gate]
        y = act(g) * u
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def skinny8_linear(x: torch.Tensor, w8, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                   gate: Optional[str] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [M <= 64, K]`` times an int8 weight with one scale per output (``quant.Int8Weight``, ``[K, N]``) ->
    ``[M, N]``; with ``gate`` the weight's outputs are ``[gate | up]`` and the result is ``act(gate) * up`` ``[M, N / 2]``.
    The kernel reads the codes in their K-major copy (``Int8Weight.kmajor``) and expands them in shared memory."""
    M, K = x.shape
    n_out = w8.cols // 2 if gate is not None else w8.cols
    if not (x.is_cuda and x.dtype == torch.bfloat16 and M <= 64 and K % 16 == 0 and K == w8.rows
            and (gate is None or (gate in _KINDS and n_out % 8 == 0))):
        res = skinny8_reference(x, w8, bias, residual, gate)
        if out is not None:
            out.copy_(res)
            return out
        return res
    from ._util import ptr, stream_ptr
    codes = w8.kmajor()
    x = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 else x.contiguous()
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, n_out) and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == w8.cols
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, n_out) and residual.stride(1) == 1
    rc = _native.lib().idrak_skinny8_gemm(x.data_ptr(), x.stride(0), codes.data_ptr(), codes.stride(0), w8.scales.data_ptr(),
                                          out.data_ptr(), out.stride(0), M, n_out, K, ptr(bias), ptr(residual),
                                          residual.stride(0) if residual is not None else 0,
                                          _KINDS[gate] if gate is not None else -1, stream_ptr())
    _native.check(rc, "idrak_skinny8_gemm")
    return out
