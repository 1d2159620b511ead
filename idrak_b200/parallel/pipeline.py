"""Pipeline parallelism: the decoder's layers cut into stages, micro-batches flowing through them (GPipe or 1F1B).

Ranks are laid out as ``stages x replicas``: rank ``= replica * stages + stage``. Stage 0 owns the embedding, the
last stage the final norm, the head and the loss; activations and their gradients cross stage boundaries with
point-to-point sends (NCCL on GPUs, gloo on CPU ranks). With tied embeddings the first and the last stage both
hold the table and sum its two gradients after backward. Replicas of a stage average their gradients. Every stage
runs its own AdamW; the clip factor comes from the gradient norm over all stages.

Schedules: ``gpipe`` - every micro-batch forward, then every backward in reverse (bubble (S-1)/(M+S-1), all M
activations held); ``1f1b`` - the same bubble, at most S - stage micro-batches in flight.

Reference: pipeline placement and GPipeSchedule (src/Idrak.Network/Training/PipelineSchedules.cs:6-40),
PipelinePretraining (src/Idrak.Text/PipelinePretraining.cs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..models.decoder import Decoder

FORWARD, BACKWARD = "F", "B"


def schedule_order(name: str, stage: int, stages: int, micro_batches: int) -> List[Tuple[str, int]]:
    """The (kind, micro-batch) work list of one stage."""
    if not (0 <= stage < stages) or micro_batches < 1:
        raise ValueError("stage must be in [0, stages) and there must be at least one micro-batch")
    if name == "gpipe":
        return [(FORWARD, m) for m in range(micro_batches)] + [(BACKWARD, m) for m in reversed(range(micro_batches))]
    if name == "1f1b":
        warm = min(stages - 1 - stage, micro_batches)
        order = [(FORWARD, m) for m in range(warm)]
        f, b = warm, 0
        while b < micro_batches:
            if f < micro_batches:
                order.append((FORWARD, f))
                f += 1
            order.append((BACKWARD, b))
            b += 1
        return order
    raise KeyError(f"Pipeline schedule '{name}' is not registered. Known: gpipe, 1f1b")


def ideal_bubble(stages: int, micro_batches: int) -> float:
    return (stages - 1.0) / (micro_batches + stages - 1.0)


def in_flight(name: str, stage: int, stages: int, micro_batches: int) -> int:
    """Most micro-batches whose activations a stage holds at once."""
    held = most = 0
    for kind, _ in schedule_order(name, stage, stages, micro_batches):
        held += 1 if kind == FORWARD else -1
        most = max(most, held)
    return most


def split_layers(layers: int, stages: int) -> List[Tuple[int, int]]:
    """Contiguous layer ranges, as even as possible (earlier stages take the extra layer)."""
    if stages > layers:
        raise ValueError(f"{stages} stages for {layers} layers")
    base, extra = divmod(layers, stages)
    out, lo = [], 0
    for s in range(stages):
        hi = lo + base + (1 if s < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


class PipelineStage(nn.Module):
    """The slice of a decoder one stage runs."""

    def __init__(self, model: Decoder, stage: int, stages: int):
        super().__init__()
        self.spec, self.stage, self.stages = model.spec, stage, stages
        lo, hi = split_layers(model.spec.layers, stages)[stage]
        self.first, self.last = stage == 0, stage == stages - 1
        self.blocks = nn.ModuleList(list(model.blocks[lo:hi]))
        self.embed = model.embed if (self.first or (self.last and model.spec.tie_embeddings)) else None
        self.pos = model.pos if self.first else None
        self.norm = model.norm if self.last else None
        self.head = model.head if (self.last and not model.spec.tie_embeddings) else None
        self.loss_chunk_rows = getattr(model, "loss_chunk_rows", None)

    def forward_hidden(self, x: torch.Tensor, ids: Optional[torch.Tensor]) -> torch.Tensor:
        if self.first:
            x = ops.embedding(ids, self.embed, self.pos)
            if self.spec.embedding_scale is not None:
                x = x * self.spec.embedding_scale
        for blk in self.blocks:
            x = blk(x)
        return x

    def loss(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        h = self.norm(x)
        w = self.embed if self.head is None else self.head
        return ops.token_cross_entropy(h, w, targets, self.spec.vocabulary, self.loss_chunk_rows, None)


@dataclass
class PipelineLayout:
    stages: int
    replicas: int
    stage: int
    replica: int

    @staticmethod
    def of(rank: int, world: int, stages: int) -> "PipelineLayout":
        if world % stages:
            raise ValueError(f"world size {world} does not divide into {stages} stages")
        return PipelineLayout(stages, world // stages, rank % stages, rank // stages)

    def rank_of(self, stage: int) -> int:
        return self.replica * self.stages + stage


class PipelineTrainer:
    def __init__(self, model: Decoder, stages: int, micro_batches: int, schedule: str = "gpipe", lr: float = 3e-4,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0, betas=(0.9, 0.95)):
        assert dist.is_initialized(), "torch.distributed must be initialised"
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.layout = PipelineLayout.of(self.rank, self.world, stages)
        self.micro_batches, self.schedule = micro_batches, schedule
        self.part = PipelineStage(model, self.layout.stage, stages)
        self.device = next(self.part.parameters()).device
        self.dtype = next(self.part.parameters()).dtype
        self.spec = model.spec
        lay = self.layout
        # groups: every rank creates every group in the same order
        self.replica_groups = [dist.new_group([r * stages + s for r in range(lay.replicas)]) for s in range(stages)]
        self.pipeline_groups = [dist.new_group([r * stages + s for s in range(stages)]) for r in range(lay.replicas)]
        self.tie_groups = [dist.new_group([r * stages, r * stages + stages - 1]) if stages > 1 else None
                           for r in range(lay.replicas)]
        params = [p for p in self.part.parameters() if p.requires_grad]
        decay = [p for p in params if p.dim() >= 2]
        rest = [p for p in params if p.dim() < 2]
        self.params = params
        self.optimizer = ops.FusedAdamW([{"params": decay, "weight_decay": weight_decay},
                                         {"params": rest, "weight_decay": 0.0}], lr=lr, betas=betas,
                                        weight_decay=weight_decay, max_grad_norm=max_grad_norm)
        self.order = schedule_order(schedule, lay.stage, stages, micro_batches)
        self._pending = []

    # ------------------------------------------------------------------ boundaries
    def _send(self, t: torch.Tensor, stage: int) -> None:
        # non-blocking: under 1F1B two neighbours may send to each other at the same moment
        t = t.contiguous()
        self._pending.append((dist.isend(t, dst=self.layout.rank_of(stage)), t))

    def _drain_sends(self) -> None:
        for req, _ in self._pending:
            req.wait()
        self._pending = []

    def _recv(self, shape, stage: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=self.dtype, device=self.device)
        dist.recv(t, src=self.layout.rank_of(stage))
        return t

    # ------------------------------------------------------------------ one step
    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> float:
        """``ids`` / ``targets``: this replica's batch ``[B, S]`` (every stage of the replica passes the same)."""
        lay, part, M = self.layout, self.part, self.micro_batches
        B, S = ids.shape
        if B % M:
            raise ValueError(f"the batch ({B}) must divide into {M} micro-batches")
        mb = B // M
        ids_m = ids.to(self.device).int().chunk(M)
        tgt_m = targets.to(self.device).int().chunk(M)
        self.optimizer.zero_grad()
        inputs, outputs = {}, {}
        loss_sum = torch.zeros((), device=self.device)
        shape = (mb, S, self.spec.dim)
        for kind, m in self.order:
            if kind == FORWARD:
                x = None
                if not part.first:
                    x = self._recv(shape, lay.stage - 1).requires_grad_(True)
                    inputs[m] = x
                h = part.forward_hidden(x, ids_m[m])
                if part.last:
                    loss = part.loss(h, tgt_m[m]) / M
                    outputs[m] = loss
                    loss_sum += loss.detach().float()
                else:
                    outputs[m] = h
                    self._send(h.detach(), lay.stage + 1)
            else:
                out = outputs.pop(m)
                if part.last:
                    out.backward()
                else:
                    out.backward(self._recv(shape, lay.stage + 1))
                if not part.first:
                    self._send(inputs.pop(m).grad, lay.stage - 1)
        self._drain_sends()
        self._finish_gradients()
        # every rank of the replica reports the step's loss (it lives on the last stage)
        if lay.stages > 1:
            dist.broadcast(loss_sum, src=lay.rank_of(lay.stages - 1), group=self.pipeline_groups[lay.replica])
        if lay.replicas > 1:
            dist.all_reduce(loss_sum, group=self.replica_groups[lay.stage])
            loss_sum /= lay.replicas
        return float(loss_sum.item())

    @torch.no_grad()
    def _finish_gradients(self) -> None:
        lay, part = self.layout, self.part
        # tied embedding: its gradient is the sum of the lookup's (first stage) and the head's (last stage)
        if self.spec.tie_embeddings and lay.stages > 1 and (part.first or part.last):
            g = part.embed.grad
            if g is None:
                g = part.embed.grad = torch.zeros_like(part.embed)
            dist.all_reduce(g, group=self.tie_groups[lay.replica])
        if lay.replicas > 1:
            flat = torch.cat([p.grad.reshape(-1).float() for p in self.params if p.grad is not None])
            dist.all_reduce(flat, group=self.replica_groups[lay.stage])
            flat /= lay.replicas
            off = 0
            for p in self.params:
                if p.grad is not None:
                    p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
                    off += p.numel()
        # global norm over the stages of this replica (a tied table is counted once: on the first stage)
        own = [p for p in self.params if not (self.spec.tie_embeddings and part.last and lay.stages > 1 and p is part.embed)]
        sq = sum((p.grad.float().pow(2).sum() for p in own if p.grad is not None), torch.zeros((), device=self.device))
        local_all = sum((p.grad.float().pow(2).sum() for p in self.params if p.grad is not None),
                        torch.zeros((), device=self.device))
        total = sq.clone()
        if lay.stages > 1:
            dist.all_reduce(total, group=self.pipeline_groups[lay.replica])
        extra = (total - local_all).reshape(1).float()
        self.optimizer.step(extra_sumsq=extra)

    # ------------------------------------------------------------------ checkpoints
    def stage_state(self) -> dict:
        """This stage's tensors under ``pipeline.<stage>.`` (the prefix the optimizer file of pipeline runs uses)."""
        pre = f"pipeline.{self.layout.stage}."
        return {pre + n: p.detach().cpu() for n, p in self.part.named_parameters()}
