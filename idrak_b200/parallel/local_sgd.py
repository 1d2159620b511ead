"""Local SGD: every rank steps on its own gradients; the weights are averaged every ``sync_every`` steps.

Between synchronisations nothing crosses the links. At a synchronisation the ranks either average their weights
(plain local SGD) or - with an outer optimizer - treat the averaged change since the last synchronisation as a
gradient and apply Nesterov momentum to it, which keeps long intervals stable. Optimizer moments stay local.

Reference: "local-sgd" gradient sync (src/Idrak.Network/Training/LocalSgd.cs:11).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class LocalSGD:
    def __init__(self, params, optimizer, sync_every: int = 16, group=None, outer_lr: float = 1.0,
                 outer_momentum: float = 0.0, compressor=None):
        if sync_every < 1:
            raise ValueError("sync_every must be at least 1")
        self.params: List[torch.Tensor] = [p for p in params if p.requires_grad]
        self.optimizer, self.sync_every, self.group = optimizer, sync_every, group
        self.outer_lr, self.outer_momentum = outer_lr, outer_momentum
        self.compressor = compressor
        self.local_steps = 0
        self.syncs = 0
        self._anchor: Optional[List[torch.Tensor]] = None      # weights at the last synchronisation
        self._velocity: Optional[List[torch.Tensor]] = None
        if outer_momentum > 0 or outer_lr != 1.0 or compressor is not None:
            self._anchor = [p.detach().float().clone() for p in self.params]

    def step(self) -> bool:
        """One local optimizer step; returns True when it ended with a synchronisation."""
        self.optimizer.step()
        self.local_steps += 1
        if self.local_steps % self.sync_every:
            return False
        self.synchronize()
        return True

    @torch.no_grad()
    def synchronize(self) -> None:
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.syncs += 1
        if self._anchor is None:
            # plain averaging of the weights, in one flat message
            flat = torch.cat([p.detach().float().reshape(-1) for p in self.params])
            if world > 1:
                dist.all_reduce(flat, group=self.group)
                flat /= world
            self._scatter(flat)
            return
        # outer step on the averaged change since the anchor
        delta = torch.cat([(a - p.detach().float()).reshape(-1) for a, p in zip(self._anchor, self.params)])
        if self.compressor is not None:
            delta = self.compressor.reduce("local-sgd", delta / world)
        elif world > 1:
            dist.all_reduce(delta, group=self.group)
            delta /= world
        if self.outer_momentum > 0:
            if self._velocity is None:
                self._velocity = [torch.zeros_like(a) for a in self._anchor]
        off = 0
        for i, (a, p) in enumerate(zip(self._anchor, self.params)):
            g = delta[off: off + a.numel()].view_as(a)
            off += a.numel()
            if self.outer_momentum > 0:
                v = self._velocity[i]
                v.mul_(self.outer_momentum).add_(g)
                g = g + self.outer_momentum * v                # Nesterov
            a.sub_(g, alpha=self.outer_lr)
            p.copy_(a.to(p.dtype))
        self._refresh_master()

    def _scatter(self, flat: torch.Tensor) -> None:
        off = 0
        for p in self.params:
            p.copy_(flat[off: off + p.numel()].view_as(p).to(p.dtype))
            off += p.numel()
        self._refresh_master()

    def _refresh_master(self) -> None:
        sync = getattr(self.optimizer, "sync_master_from_params", None)
        if callable(sync):
            sync()
