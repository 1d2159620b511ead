"""Knowledge distillation of a decoder: the student learns from a mix of the data's next-token loss and the teacher's
softened distribution. Teacher outputs can be computed on the fly or read from a cache that keeps the top-k
log-probabilities per position (what makes distilling from a large teacher affordable).

    d = Distiller(student, teacher, optimizer, alpha=0.5, temperature=2.0)
    for ids in batches:
        stats = d.step(ids)

Reference: src/Idrak.Text/Distillation.cs (loss mix, temperature, masks) and TeacherLogits (top-k cache files).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..formats.safetensors import load_file, save_file


@dataclass
class TeacherTopK:
    """Top-k teacher log-probabilities per position: ``indices`` / ``values`` ``[N, T, k]`` and the log of the mass
    left outside the top k (``rest`` ``[N, T]``), spread evenly over the other tokens when the loss needs it."""
    indices: torch.Tensor
    values: torch.Tensor
    rest: torch.Tensor

    @classmethod
    @torch.no_grad()
    def from_logits(cls, logits: torch.Tensor, k: int = 32, temperature: float = 1.0) -> "TeacherTopK":
        lp = F.log_softmax(logits.float() / temperature, -1)
        top = lp.topk(min(k, lp.shape[-1]), -1)
        mass = top.values.exp().sum(-1).clamp(max=1.0 - 1e-7)
        return cls(top.indices.to(torch.int32), top.values.to(torch.float16), torch.log1p(-mass).to(torch.float16))

    def save(self, path: str) -> None:
        save_file({"indices": self.indices.cpu(), "values": self.values.cpu(), "rest": self.rest.cpu()}, path,
                  metadata={"format": "idrak-teacher-topk/1"})

    @classmethod
    def load(cls, path: str) -> "TeacherTopK":
        t = load_file(path)
        return cls(t["indices"], t["values"], t["rest"])


def topk_distillation_loss(student_logits: torch.Tensor, teacher: TeacherTopK, temperature: float = 1.0,
                           mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Cross-entropy of the student (at the temperature) against the teacher's top-k distribution, with the teacher's
    remaining mass matched against the student's remaining mass; equals the full KL up to the teacher's entropy when
    k covers the vocabulary. Scaled by T^2."""
    ls = F.log_softmax(student_logits.float() / temperature, -1)
    idx = teacher.indices.long().to(ls.device)
    tv = teacher.values.float().to(ls.device)
    picked = ls.gather(-1, idx)
    loss = -(tv.exp() * picked).sum(-1)
    rest_t = teacher.rest.float().to(ls.device).exp()
    rest_s = torch.log1p(-picked.exp().sum(-1).clamp(max=1.0 - 1e-6))
    loss = loss - rest_t * rest_s
    if mask is not None:
        m = mask.float().to(ls.device)
        return (loss * m).sum() / m.sum().clamp_min(1.0) * temperature * temperature
    return loss.mean() * temperature * temperature


class Distiller:
    def __init__(self, student, teacher, optimizer, alpha: float = 0.5, temperature: float = 2.0, top_k: int = 0,
                 max_grad_norm: float = 1.0):
        """``alpha`` weighs the data loss, ``1 - alpha`` the teacher term. ``top_k > 0`` distils from the teacher's top-k
        only (the cached form)."""
        self.student, self.teacher, self.opt = student, teacher, optimizer
        self.alpha, self.temperature, self.top_k, self.max_grad_norm = alpha, temperature, top_k, max_grad_norm
        if teacher is not None:
            teacher.eval()
            for p in teacher.parameters():
                p.requires_grad_(False)

    def loss(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None, cached: Optional[TeacherTopK] = None):
        x, y = ids[:, :-1], ids[:, 1:]
        m = mask[:, 1:] if mask is not None else None
        logits = self.student(x).float()
        V = logits.shape[-1]
        ce = F.cross_entropy(logits.reshape(-1, V), y.reshape(-1).long(), reduction="none").view_as(y)
        ce = (ce * m.float()).sum() / m.float().sum().clamp_min(1.0) if m is not None else ce.mean()
        T = self.temperature
        if cached is not None:
            kd = topk_distillation_loss(logits, cached, T, m)
        else:
            with torch.no_grad():
                t_logits = self.teacher(x).float()[..., :V]
            if self.top_k:
                kd = topk_distillation_loss(logits, TeacherTopK.from_logits(t_logits, self.top_k, T), T, m)
            else:
                from ..nn.losses import distillation_kl
                kd = distillation_kl(logits, t_logits, T, m)
        return self.alpha * ce + (1 - self.alpha) * kd, {"data_loss": float(ce.detach()), "teacher_loss": float(kd.detach())}

    def step(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None, cached: Optional[TeacherTopK] = None) -> Dict[str, float]:
        self.student.train()
        loss, stats = self.loss(ids, mask, cached)
        self.opt.zero_grad()
        loss.backward()
        if self.max_grad_norm:
            stats["grad_norm"] = float(torch.nn.utils.clip_grad_norm_(self.student.parameters(), self.max_grad_norm))
        self.opt.step()
        stats["loss"] = float(loss.detach())
        return stats
