"""Connectionist temporal classification loss on the device (``csrc/ctc.cu``), with the PyTorch statement for the CPU.

``ctc_loss(log_probs, targets, input_lengths, target_lengths)`` takes log-probabilities ``[T, B, C]`` (the output of a
log-softmax), padded targets ``[B, L]`` and the two length vectors, and returns the negative log-likelihood of every
sequence ``[B]``; reductions are the caller's (``nn.losses.CTCLoss`` applies them). The gradient is the true derivative
with respect to the log-probabilities, so it composes with any normalisation in front of it.

Reference: Tensor.CtcLoss (src/Idrak.Abstraction/Tensors/Tensor.Ctc.cs), ctc_loss_f32 / ctc_loss_bwd_f32
(src/Idrak.Gpu/Cuda/PtxKernels.Ctc.cs).
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import stream_ptr

NO_ALIGNMENT = 3.4028234663852886e38          # what the kernel writes when no path exists


def ctc_reference(log_probs, targets, input_lengths, target_lengths, blank=0):
    """Per-sequence negative log-likelihood by PyTorch (``inf`` where no alignment exists)."""
    return torch.nn.functional.ctc_loss(log_probs.float(), targets.long(), input_lengths.long(), target_lengths.long(),
                                        blank=blank, reduction="none", zero_infinity=False)


class _Ctc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, log_probs, targets, input_lengths, target_lengths, blank):
        T, B, Cn = log_probs.shape
        L = targets.shape[1]
        lib = _native.lib()
        dev = log_probs.device
        alpha = torch.empty(lib.idrak_ctc_alpha_elems(T, B, L), dtype=torch.float32, device=dev)
        rows = torch.empty(lib.idrak_ctc_row_elems(B, L), dtype=torch.float32, device=dev)
        loss = torch.empty(B, dtype=torch.float32, device=dev)
        rc = lib.idrak_ctc_loss(log_probs.data_ptr(), targets.data_ptr(), input_lengths.data_ptr(),
                                target_lengths.data_ptr(), alpha.data_ptr(), rows.data_ptr(), loss.data_ptr(), T, B, Cn,
                                L, blank, stream_ptr())
        _native.check(rc, "idrak_ctc_loss")
        ctx.save_for_backward(log_probs, targets, input_lengths, target_lengths, alpha, loss)
        ctx.blank = blank
        return torch.where(loss >= NO_ALIGNMENT, torch.full_like(loss, float("inf")), loss)

    @staticmethod
    def backward(ctx, grad_out):
        log_probs, targets, input_lengths, target_lengths, alpha, loss = ctx.saved_tensors
        T, B, Cn = log_probs.shape
        L = targets.shape[1]
        lib = _native.lib()
        dev = log_probs.device
        rows = torch.empty(lib.idrak_ctc_row_elems(B, L), dtype=torch.float32, device=dev)
        chain = torch.empty(B * (2 * L + 1), dtype=torch.int32, device=dev)
        grad = torch.empty_like(log_probs)
        go = grad_out.to(torch.float32).contiguous()
        rc = lib.idrak_ctc_loss_bwd(log_probs.data_ptr(), targets.data_ptr(), input_lengths.data_ptr(),
                                    target_lengths.data_ptr(), alpha.data_ptr(), loss.data_ptr(), go.data_ptr(),
                                    rows.data_ptr(), chain.data_ptr(), grad.data_ptr(), T, B, Cn, L, ctx.blank,
                                    stream_ptr())
        _native.check(rc, "idrak_ctc_loss_bwd")
        return grad, None, None, None, None


def ctc_loss(log_probs: torch.Tensor, targets: torch.Tensor, input_lengths: torch.Tensor,
             target_lengths: torch.Tensor, blank: int = 0) -> torch.Tensor:
    """Negative log-likelihood per sequence, ``[B]`` fp32; ``inf`` (and a zero gradient) where no alignment exists."""
    if log_probs.dim() != 3 or targets.dim() != 2:
        raise ValueError("ctc_loss takes log_probs [T, B, C] and padded targets [B, L]")
    if not log_probs.is_cuda:
        return ctc_reference(log_probs, targets, input_lengths, target_lengths, blank)
    dev = log_probs.device
    lp = log_probs.float().contiguous()
    tg = targets.to(device=dev, dtype=torch.int32).contiguous()
    if tg.shape[1] == 0:
        tg = torch.zeros((tg.shape[0], 1), dtype=torch.int32, device=dev)
    il = input_lengths.to(device=dev, dtype=torch.int32).contiguous()
    tl = target_lengths.to(device=dev, dtype=torch.int32).contiguous()
    return _Ctc.apply(lp, tg, il, tl, int(blank))
