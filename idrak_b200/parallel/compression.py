"""Gradient compression for data-parallel reductions over slow links: what travels is smaller than fp32, what the
optimizer sees is still the sum over ranks.

Kinds (by name, as in the reference's GradientCompressions): ``none`` (fp32), ``bf16`` (half the bytes, sums in
fp32), ``int8`` and ``fp8`` (one byte per value times a per-piece scale), ``top-k`` (only the largest share of each
bucket by magnitude, as index / value pairs). With error feedback a rank adds what it did not send to its next
step's values, so nothing is lost, only late. Sums are made in rank order, so every rank holds the same bits.

Inside one NVSwitch domain the fused bf16 path (``parallel/dp.py``) is faster than any of these; they are for
links between nodes. Reference: src/Idrak.Network/Compression/{Compressions,Quantized,TopK}.cs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

PIECE = 4096            # values sharing one scale in the int8 / fp8 compressions
KINDS = ("none", "bf16", "int8", "fp8", "top-k")


def _gather(t: torch.Tensor, group) -> List[torch.Tensor]:
    world = dist.get_world_size(group)
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


class Compressor:
    """``reduce(name, flat)`` replaces ``flat`` (fp32, this rank's weighted gradient bucket) by the sum over ranks."""

    def __init__(self, kind: str = "none", group=None, error_feedback: bool = True, top_k: float = 0.01):
        if kind not in KINDS:
            raise KeyError(f"Gradient compression '{kind}' is not registered. Known: {', '.join(KINDS)}")
        if not (0.0 < top_k <= 1.0):
            raise ValueError("top_k is a share of the values, in (0, 1]")
        self.kind, self.group, self.error_feedback, self.top_k = kind, group, error_feedback, top_k
        self.residual: Dict[str, torch.Tensor] = {}
        self.bytes_sent = 0
        self.bytes_dense = 0

    # ------------------------------------------------------------------ helpers
    def _with_residual(self, name: str, flat: torch.Tensor) -> torch.Tensor:
        if self.error_feedback and name in self.residual:
            flat = flat + self.residual[name]
        return flat

    def _keep_residual(self, name: str, wanted: torch.Tensor, sent: torch.Tensor) -> None:
        if self.error_feedback:
            self.residual[name] = wanted - sent

    # ------------------------------------------------------------------ kinds
    def reduce(self, name: str, flat: torch.Tensor) -> torch.Tensor:
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.bytes_dense += flat.numel() * 4
        if world == 1 and self.kind in ("none", "bf16"):
            return flat
        if self.kind == "none":
            self.bytes_sent += flat.numel() * 4
            parts = _gather(flat, self.group)
            return self._ordered_sum(parts)
        if self.kind == "bf16":
            self.bytes_sent += flat.numel() * 2
            parts = _gather(flat.to(torch.bfloat16), self.group)
            return self._ordered_sum([p.float() for p in parts])
        if self.kind in ("int8", "fp8"):
            return self._quantized(name, flat, world)
        return self._topk(name, flat, world)

    @staticmethod
    def _ordered_sum(parts: List[torch.Tensor]) -> torch.Tensor:
        total = parts[0].clone()
        for p in parts[1:]:
            total += p                   # rank order: the same bits on every rank
        return total

    def _quantized(self, name: str, flat: torch.Tensor, world: int) -> torch.Tensor:
        want = self._with_residual(name, flat)
        n = want.numel()
        pieces = (n + PIECE - 1) // PIECE
        padded = torch.zeros(pieces * PIECE, dtype=torch.float32, device=want.device)
        padded[:n] = want
        view = padded.view(pieces, PIECE)
        amax = view.abs().amax(dim=1).clamp_min(1e-30)
        if self.kind == "int8":
            scale = amax / 127.0
            codes = torch.round(view / scale[:, None]).clamp_(-127, 127).to(torch.int8)
            sent = codes.float() * scale[:, None]
            payload = codes
        else:
            scale = amax / 448.0
            payload = (view / scale[:, None]).to(torch.float8_e4m3fn)
            sent = payload.float() * scale[:, None]
        self._keep_residual(name, want, sent.view(-1)[:n])
        self.bytes_sent += payload.numel() + scale.numel() * 4
        if world == 1:
            return sent.view(-1)[:n].clone()
        raw = payload.view(torch.uint8) if payload.dtype != torch.int8 else payload
        all_codes, all_scales = _gather(raw, self.group), _gather(scale, self.group)
        total = torch.zeros(pieces, PIECE, dtype=torch.float32, device=want.device)
        for c, s in zip(all_codes, all_scales):
            vals = c.float() if self.kind == "int8" else c.view(torch.float8_e4m3fn).float()
            total += vals * s[:, None]
        return total.view(-1)[:n].clone()

    def _topk(self, name: str, flat: torch.Tensor, world: int) -> torch.Tensor:
        want = self._with_residual(name, flat)
        n = want.numel()
        k = max(1, int(math.ceil(n * self.top_k)))
        # ties go to the lower index: sort by (-|v|, index) through a stable sort on the magnitudes
        order = torch.sort(want.abs(), descending=True, stable=True).indices[:k]
        idx = torch.sort(order).values
        vals = want[idx]
        sent = torch.zeros_like(want)
        sent[idx] = vals
        self._keep_residual(name, want, sent)
        self.bytes_sent += k * 8
        if world == 1:
            return sent
        all_idx, all_vals = _gather(idx.to(torch.int64), self.group), _gather(vals, self.group)
        total = torch.zeros_like(want)
        for i, v in zip(all_idx, all_vals):
            total.index_add_(0, i, v)
        return total

    def ratio(self) -> float:
        return self.bytes_sent / self.bytes_dense if self.bytes_dense else 1.0


class CompressedGradientReducer:
    """Data-parallel gradient averaging through a ``Compressor``: parameters are cut into buckets in backward order
    (the order their gradients become ready), each bucket is weighted by this rank's share and summed over ranks."""

    def __init__(self, params, kind: str = "none", group=None, bucket_elems: int = 1 << 22, error_feedback: bool = True,
                 top_k: float = 0.01):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.compressor = Compressor(kind, group, error_feedback, top_k)
        self.buckets: List[List[int]] = []
        cur, size = [], 0
        for i in reversed(range(len(self.params))):
            cur.append(i)
            size += self.params[i].numel()
            if size >= bucket_elems:
                self.buckets.append(cur)
                cur, size = [], 0
        if cur:
            self.buckets.append(cur)

    @torch.no_grad()
    def reduce(self, weight: Optional[float] = None) -> None:
        """Replace every ``p.grad`` by the weighted sum over ranks (``weight`` defaults to 1 / world: the mean)."""
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        w = (1.0 / world) if weight is None else weight
        for b, members in enumerate(self.buckets):
            grads = [self.params[i].grad for i in members]
            if any(g is None for g in grads):
                raise RuntimeError("a parameter of the bucket has no gradient; freeze it or exclude it")
            flat = torch.cat([g.reshape(-1).float() for g in grads]) * w
            total = self.compressor.reduce(f"bucket{b}", flat)
            off = 0
            for g in grads:
                g.copy_(total[off: off + g.numel()].view_as(g))
                off += g.numel()
