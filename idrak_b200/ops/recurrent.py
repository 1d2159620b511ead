"""LSTM and GRU: cell arithmetic on the device (``csrc/recurrent.cu``) and the sequence drivers built on it.

A layer over a sequence runs the input projection of all time steps as one many-row product, then per step one few-row
product with the hidden weights and one cell launch. bf16 tensors take the tcgen05 GEMM for the products; fp32 tensors
use the library product (the cell kernels are the same). Gate order and arithmetic follow ``torch.nn.LSTM`` /
``torch.nn.GRU``, so their weights load unchanged, and the CPU path is those formulas in plain PyTorch.

Reference: Lstm / Gru layers (src/Idrak/Layers/Recurrent.cs) and lstm_cell / gru_cell (+bwd)
(src/Idrak.Gpu/Cuda/PtxKernels.Recurrent.cs).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import _native
from ._util import ptr, stream_ptr

_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def _ok(*ts) -> bool:
    t0 = ts[0]
    return t0.is_cuda and t0.dtype in _DTYPES and all(t.is_cuda and t.dtype == t0.dtype for t in ts)


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


# ------------------------------------------------------------------------------------------------------------ references
def lstm_cell_reference(gates, c_prev):
    i, f, g, o = gates.float().chunk(4, -1)
    c = torch.sigmoid(f) * c_prev.float() + torch.sigmoid(i) * torch.tanh(g)
    h = torch.sigmoid(o) * torch.tanh(c)
    return h.to(gates.dtype), c.to(gates.dtype)


def gru_cell_reference(gi, gh, h_prev):
    ir, iz, inn = gi.float().chunk(3, -1)
    hr, hz, hn = gh.float().chunk(3, -1)
    r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
    n = torch.tanh(inn + r * hn)
    return ((1 - z) * n + z * h_prev.float()).to(gi.dtype)


# ----------------------------------------------------------------------------------------------------------------- cells
class _LstmCell(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, c_prev):
        B, H4 = gates.shape
        H = H4 // 4
        h, c = torch.empty_like(c_prev), torch.empty_like(c_prev)
        acts = torch.empty_like(gates)
        rc = _native.lib().idrak_lstm_cell(_DTYPES[gates.dtype], gates.data_ptr(), c_prev.data_ptr(), h.data_ptr(),
                                           c.data_ptr(), acts.data_ptr(), B, H, stream_ptr())
        _native.check(rc, "idrak_lstm_cell")
        ctx.save_for_backward(acts, c_prev, c)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        acts, c_prev, c = ctx.saved_tensors
        B, H = c.shape
        dh = _c(dh) if dh is not None else torch.zeros_like(c)
        dc = _c(dc) if dc is not None else None
        dgates, dc_prev = torch.empty_like(acts), torch.empty_like(c)
        rc = _native.lib().idrak_lstm_cell_bwd(_DTYPES[c.dtype], acts.data_ptr(), c_prev.data_ptr(), c.data_ptr(),
                                               dh.data_ptr(), ptr(dc), dgates.data_ptr(), dc_prev.data_ptr(), B, H,
                                               stream_ptr())
        _native.check(rc, "idrak_lstm_cell_bwd")
        return dgates, dc_prev


def lstm_cell(gates: torch.Tensor, c_prev: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gates`` ``[B, 4H]``: the summed projections and biases in (input, forget, cell, output) order. Returns
    ``(h, c)``."""
    if not _ok(gates, c_prev):
        return lstm_cell_reference(gates, c_prev)
    return _LstmCell.apply(_c(gates), _c(c_prev))


class _GruCell(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gi, gh, h_prev):
        B, H3 = gi.shape
        H = H3 // 3
        h = torch.empty_like(h_prev)
        acts = torch.empty((B, 4 * H), dtype=gi.dtype, device=gi.device)
        rc = _native.lib().idrak_gru_cell(_DTYPES[gi.dtype], gi.data_ptr(), gh.data_ptr(), h_prev.data_ptr(),
                                          h.data_ptr(), acts.data_ptr(), B, H, stream_ptr())
        _native.check(rc, "idrak_gru_cell")
        ctx.save_for_backward(acts, h_prev)
        return h

    @staticmethod
    def backward(ctx, dh):
        acts, h_prev = ctx.saved_tensors
        B, H = h_prev.shape
        dh = _c(dh)
        dgi = torch.empty((B, 3 * H), dtype=dh.dtype, device=dh.device)
        dgh = torch.empty_like(dgi)
        dhp = torch.empty_like(h_prev)
        rc = _native.lib().idrak_gru_cell_bwd(_DTYPES[dh.dtype], acts.data_ptr(), h_prev.data_ptr(), dh.data_ptr(),
                                              dgi.data_ptr(), dgh.data_ptr(), dhp.data_ptr(), B, H, stream_ptr())
        _native.check(rc, "idrak_gru_cell_bwd")
        return dgi, dgh, dhp


def gru_cell(gi: torch.Tensor, gh: torch.Tensor, h_prev: torch.Tensor) -> torch.Tensor:
    """``gi`` / ``gh`` ``[B, 3H]``: input and hidden projections (with their biases) in (reset, update, new) order."""
    if not _ok(gi, gh, h_prev):
        return gru_cell_reference(gi, gh, h_prev)
    return _GruCell.apply(_c(gi), _c(gh), _c(h_prev))


# ------------------------------------------------------------------------------------------------------------- sequences
def _project(x2, weight, bias):
    """``x2 @ weight.T + bias``: the tcgen05 GEMM for bf16 with 16-byte rows, the library product otherwise."""
    if x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        from .gemm import linear
        return linear(x2, weight.to(x2.dtype), None if bias is None else bias.to(x2.dtype))
    return F.linear(x2, weight.to(x2.dtype), None if bias is None else bias.to(x2.dtype))


def lstm_layer(x: torch.Tensor, w_ih, w_hh, b_ih=None, b_hh=None, state: Optional[Tuple] = None,
               reverse: bool = False):
    """One direction of one LSTM layer over ``x`` ``[T, B, in]``. Returns ``(outputs [T, B, H], (h_T, c_T))``."""
    T, B, _ = x.shape
    H = w_hh.shape[1]
    bias = b_ih if b_hh is None else (b_hh if b_ih is None else b_ih + b_hh)
    xi = _project(x.reshape(T * B, -1), w_ih, bias).reshape(T, B, 4 * H)
    if state is None:
        h = torch.zeros(B, H, dtype=x.dtype, device=x.device)
        c = torch.zeros(B, H, dtype=x.dtype, device=x.device)
    else:
        h, c = state
    outs = [None] * T
    for t in (range(T - 1, -1, -1) if reverse else range(T)):
        gates = xi[t] + _project(h, w_hh, None)
        h, c = lstm_cell(gates, c)
        outs[t] = h
    return torch.stack(outs), (h, c)


def gru_layer(x: torch.Tensor, w_ih, w_hh, b_ih=None, b_hh=None, state: Optional[torch.Tensor] = None,
              reverse: bool = False):
    """One direction of one GRU layer over ``x`` ``[T, B, in]``. Returns ``(outputs [T, B, H], h_T)``."""
    T, B, _ = x.shape
    H = w_hh.shape[1]
    xi = _project(x.reshape(T * B, -1), w_ih, b_ih).reshape(T, B, 3 * H)
    h = torch.zeros(B, H, dtype=x.dtype, device=x.device) if state is None else state
    outs = [None] * T
    for t in (range(T - 1, -1, -1) if reverse else range(T)):
        h = gru_cell(xi[t], _project(h, w_hh, b_hh), h)
        outs[t] = h
    return torch.stack(outs), h


def run_module(module: torch.nn.Module, x: torch.Tensor):
    """Run a ``torch.nn.LSTM`` / ``torch.nn.GRU`` (its parameters, layer count, directions, ``batch_first``) through the
    drivers above. Returns ``(outputs, final_state)`` like the module does; dropout between layers is not applied."""
    is_lstm = isinstance(module, torch.nn.LSTM)
    if module.batch_first:
        x = x.transpose(0, 1)
    x = _c(x)
    finals_h, finals_c = [], []
    for layer in range(module.num_layers):
        outs = []
        for d in range(2 if module.bidirectional else 1):
            sfx = f"_l{layer}" + ("_reverse" if d else "")
            w_ih, w_hh = getattr(module, "weight_ih" + sfx), getattr(module, "weight_hh" + sfx)
            b_ih = getattr(module, "bias_ih" + sfx, None) if module.bias else None
            b_hh = getattr(module, "bias_hh" + sfx, None) if module.bias else None
            if is_lstm:
                o, (h, c) = lstm_layer(x, w_ih, w_hh, b_ih, b_hh, reverse=bool(d))
                finals_c.append(c)
            else:
                o, h = gru_layer(x, w_ih, w_hh, b_ih, b_hh, reverse=bool(d))
            finals_h.append(h)
            outs.append(o)
        x = outs[0] if len(outs) == 1 else torch.cat(outs, -1)
    out = x.transpose(0, 1) if module.batch_first else x
    hN = torch.stack(finals_h)
    return out, ((hN, torch.stack(finals_c)) if is_lstm else hN)
