"""Losses with the reference's names. Token cross-entropy (the head applied in row chunks with a fused softmax, so
the ``[tokens, vocabulary]`` logits never exist) lives in ``ops.token_cross_entropy``; the rest are thin, explicit
statements over tensors.

Reference: src/Idrak/Losses.cs (MSE / MAE / cross-entropy with label smoothing / sparse / pixel-wise / binary with and
without logits / TokenCrossEntropy :86-104 / TokenLogProbabilities / distillation KL / CTC / adversarial and
feature-matching terms).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from ..ops import token_cross_entropy  # noqa: F401  (re-exported)


def mse(prediction, target):
    return F.mse_loss(prediction.float(), target.float())


def mae(prediction, target):
    return F.l1_loss(prediction.float(), target.float())


def huber(prediction, target, delta: float = 1.0):
    return F.huber_loss(prediction.float(), target.float(), delta=delta)


def cross_entropy(logits, target_probabilities, label_smoothing: float = 0.0):
    """Targets as probability rows (one-hot or soft)."""
    t = target_probabilities.float()
    if label_smoothing:
        t = t * (1 - label_smoothing) + label_smoothing / t.shape[-1]
    return -(t * F.log_softmax(logits.float(), -1)).sum(-1).mean()


def sparse_cross_entropy(logits, target_ids, label_smoothing: float = 0.0, ignore_index: int = -100):
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), target_ids.reshape(-1).long(),
                           label_smoothing=label_smoothing, ignore_index=ignore_index)


def pixel_cross_entropy(logits, target_ids, ignore_index: int = -100):
    """``logits`` [N, classes, H, W], ``target_ids`` [N, H, W]."""
    return F.cross_entropy(logits.float(), target_ids.long(), ignore_index=ignore_index)


def binary_cross_entropy(probabilities, target):
    return F.binary_cross_entropy(probabilities.float().clamp(1e-7, 1 - 1e-7), target.float())


def binary_cross_entropy_with_logits(logits, target, positive_weight: Optional[torch.Tensor] = None):
    return F.binary_cross_entropy_with_logits(logits.float(), target.float(), pos_weight=positive_weight)


def token_log_probabilities(logits, target_ids):
    """Log-probability of each target token: ``[..., T, V]``, ``[..., T]`` -> ``[..., T]``."""
    return F.log_softmax(logits.float(), -1).gather(-1, target_ids.long()[..., None])[..., 0]


def distillation_kl(student_logits, teacher_logits, temperature: float = 1.0, mask: Optional[torch.Tensor] = None):
    """KL(teacher || student) at a temperature, scaled by T^2 (so gradients keep their size as T grows); ``mask``
    selects the positions that count."""
    s = F.log_softmax(student_logits.float() / temperature, -1)
    t = F.log_softmax(teacher_logits.float() / temperature, -1)
    kl = (t.exp() * (t - s)).sum(-1)
    if mask is not None:
        m = mask.float()
        return (kl * m).sum() / m.sum().clamp_min(1.0) * temperature * temperature
    return kl.mean() * temperature * temperature


def ctc(log_probabilities, targets, input_lengths, target_lengths, blank: int = 0):
    """``log_probabilities`` [T, N, classes] (log-softmax already applied)."""
    if log_probabilities.is_cuda and targets.dim() == 2:
        from ..ops.ctc import ctc_loss
        nll = ctc_loss(log_probabilities, targets, input_lengths, target_lengths, blank)      # per sequence
        nll = torch.where(torch.isinf(nll), torch.zeros_like(nll), nll)                       # no alignment: counts as 0
        return (nll / target_lengths.to(nll.device).clamp_min(1).to(nll.dtype)).mean()
    return F.ctc_loss(log_probabilities.float(), targets, input_lengths, target_lengths, blank=blank, zero_infinity=True)


def hinge_discriminator(real_scores: Sequence[torch.Tensor], fake_scores: Sequence[torch.Tensor]):
    return sum(F.relu(1 - r).mean() + F.relu(1 + f).mean() for r, f in zip(real_scores, fake_scores))


def least_squares_discriminator(real_scores, fake_scores):
    return sum(((1 - r) ** 2).mean() + (f ** 2).mean() for r, f in zip(real_scores, fake_scores))


def least_squares_generator(fake_scores):
    return sum(((1 - f) ** 2).mean() for f in fake_scores)


def feature_matching(real_features: Sequence[Sequence[torch.Tensor]], fake_features: Sequence[Sequence[torch.Tensor]]):
    """Mean absolute difference between discriminator activations on real and generated inputs."""
    total = 0.0
    for rs, fs in zip(real_features, fake_features):
        for r, f in zip(rs, fs):
            total = total + (r.detach() - f).abs().mean()
    return total


LOSSES = {"mse": mse, "mae": mae, "huber": huber, "cross_entropy": cross_entropy, "sparse_cross_entropy": sparse_cross_entropy,
          "pixel_cross_entropy": pixel_cross_entropy, "bce": binary_cross_entropy, "bce_logits": binary_cross_entropy_with_logits}
