"""Token cross-entropy: fused softmax-CE on the logits, and the chunked head + loss that never keeps the
full ``[tokens, vocab]`` logits alive.

``token_cross_entropy(hidden, head_weight, targets)`` runs the vocabulary head in row chunks; for each
chunk the GEMM writes bf16 logits, one kernel turns them into loss and (in place) gradient, and the two
gradient GEMMs of the head run at once, so the backward pass of this op only scales what is stored.

Reference: Losses.TokenCrossEntropy (src/Idrak/Losses.cs:86-104), Tensor.TokenCrossEntropy
(src/Idrak.Abstraction/Tensors/Tensor.Decoder.cs:73), softmax_ce_rows_f32.
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr
from .gemm import gemm


def softmax_xent_(logits: torch.Tensor, targets: torch.Tensor, vocab: int, grad_scale: float,
                  ignore_index: int = -100, write_grad: bool = True):
    """logits [rows, ld] bf16 (ld >= vocab, padded columns ignored). Returns per-row losses (fp32);
    when ``write_grad`` the logits are replaced by ``(softmax - onehot) * grad_scale``."""
    rows, ld = logits.shape
    t32 = targets.reshape(-1).to(torch.int32)
    if not (logits.is_cuda and logits.dtype == torch.bfloat16):
        lf = logits[:, :vocab].float()
        lse = torch.logsumexp(lf, -1)
        valid = t32 != ignore_index
        tsafe = torch.where(valid, t32, torch.zeros_like(t32)).long()
        losses = torch.where(valid, lse - lf.gather(1, tsafe[:, None])[:, 0], torch.zeros_like(lse))
        if write_grad:
            g = torch.softmax(lf, -1)
            g[torch.arange(rows), tsafe] -= 1.0
            g = g * grad_scale * valid[:, None]
            logits.zero_()
            logits[:, :vocab] = g.to(logits.dtype)
        return losses
    losses = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = _native.lib().idrak_softmax_xent(logits.data_ptr(), t32.data_ptr(), losses.data_ptr(), None, rows, vocab,
                                          logits.stride(0), float(grad_scale), ignore_index, int(write_grad),
                                          stream_ptr())
    _native.check(rc, "idrak_softmax_xent")
    return losses


class _TokenCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, vocab, chunk_rows, ignore_index):
        C = hidden.shape[-1]
        h2 = hidden.reshape(-1, C)
        if h2.stride(1) != 1 or h2.stride(0) != C:
            h2 = h2.contiguous()
        rows = h2.shape[0]
        t = targets.reshape(-1)
        # gradients are produced for d(mean loss) with upstream gradient 1; backward rescales them
        need_grad = hidden.requires_grad or weight.requires_grad
        dh = torch.empty_like(h2) if need_grad else None
        dw = None
        losses = []
        inv_dev = None
        chunk_rows = chunk_rows or rows
        if ignore_index is None:
            inv = 1.0 / rows            # every row counts: no device-to-host read
            ignore_index = -(2 ** 31)
        else:
            if torch.cuda.is_current_stream_capturing():
                # a recorded step cannot read the count back: the kernels work on sums and the division by the number
                # of rows that count stays on the device, in the loss and (through backward's rescale) in the gradients
                inv = 1.0
                inv_dev = 1.0 / (t != ignore_index).sum().clamp(min=1).float()
            else:
                inv = 1.0 / max(1, int((t != ignore_index).sum().item()))
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            logits = gemm(h2[r0:r1], weight)                       # [chunk, Vpad]
            losses.append(softmax_xent_(logits, t[r0:r1], vocab, inv, ignore_index, write_grad=need_grad))
            if need_grad:
                gemm(logits, weight, b_mn=True, out=dh[r0:r1])     # dH = dL @ W
                if dw is None:
                    dw = gemm(logits, h2[r0:r1], a_mn=True, b_mn=True, out_dtype=torch.float32)
                else:
                    gemm(logits, h2[r0:r1], a_mn=True, b_mn=True, out=dw, beta=True)
        loss = torch.cat(losses).sum() * inv
        if inv_dev is not None:
            loss = loss * inv_dev
        ctx.inv_dev = inv_dev
        ctx.save_for_backward(dh, dw)
        ctx.param = weight
        ctx.hshape, ctx.wdtype = hidden.shape, weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        from . import _grad
        dh, dw = ctx.saved_tensors
        if ctx.inv_dev is not None:
            dloss = dloss * ctx.inv_dev
        gh = (dh * dloss.to(dh.dtype)).reshape(ctx.hshape) if dh is not None and ctx.needs_input_grad[0] else None
        gw = None
        if dw is not None and ctx.needs_input_grad[1]:
            tgt = _grad.target(ctx.param)
            if tgt is not None:
                g, accumulate = tgt
                if accumulate:
                    g.add_((dw * dloss).to(g.dtype))
                else:
                    torch.mul(dw, dloss.to(dw.dtype), out=g) if g.dtype == dw.dtype else g.copy_(dw * dloss)
                _grad.written(ctx.param)
            else:
                gw = (dw * dloss).to(ctx.wdtype)
        return gh, gw, None, None, None, None


def token_cross_entropy(hidden: torch.Tensor, head_weight: torch.Tensor, targets: torch.Tensor,
                        vocab: int | None = None, chunk_rows: int | None = 8192,
                        ignore_index: int | None = -100) -> torch.Tensor:
    """Mean next-token cross-entropy of ``hidden @ head_weight^T`` against ``targets``.

    ``head_weight`` is ``[vocab_padded, dim]``; rows at and beyond ``vocab`` are padding.
    ``ignore_index=None`` states that every target counts, which keeps the step free of host reads.
    """
    vocab = vocab or head_weight.shape[0]
    if not (hidden.is_cuda and hidden.dtype == torch.bfloat16):
        logits = torch.nn.functional.linear(hidden, head_weight)[..., :vocab]
        return torch.nn.functional.cross_entropy(logits.reshape(-1, vocab).float(), targets.reshape(-1).long(),
                                                 ignore_index=-100 if ignore_index is None else ignore_index)
    return _TokenCrossEntropy.apply(hidden, head_weight, targets, vocab, chunk_rows, ignore_index)


def cross_entropy_logits(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy when the logits already exist (evaluation paths)."""
    V = logits.shape[-1]
    l2 = logits.reshape(-1, V)
    if l2.is_cuda and l2.dtype == torch.bfloat16 and V % 8 == 0 and not l2.requires_grad:
        losses = softmax_xent_(l2.contiguous(), targets, V, 0.0, ignore_index, write_grad=False)
        n = (targets.reshape(-1) != ignore_index).sum().clamp(min=1)
        return losses.sum() / n
    return torch.nn.functional.cross_entropy(l2.float(), targets.reshape(-1).long(), ignore_index=ignore_index)
