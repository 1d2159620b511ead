"""Gradient sharding ("gradients" mode of the sharded data parallel): parameters stay whole on every rank, but a
bucket's gradients are reduce-scattered as soon as the backward pass has produced them and the full gradients are
released at once, so each rank holds 1 / world of the gradients and of the optimizer state. After the optimizer has
stepped the shards, the new values are all-gathered back into the parameters.

    sharded = ShardedGradients(model, bucket_elems=1 << 22)
    opt = torch.optim.AdamW(sharded.parameters(), lr=...)        # fp32 shards (master copies)
    loss.backward(); sharded.finish_backward(); opt.step(); sharded.publish(); opt.zero_grad()

Buckets are built in reverse parameter order (the order gradients arrive in). A bucket's reduce-scatter starts from the
hook of the last gradient it waits for, asynchronously where the backend allows, so communication overlaps the rest
of the backward pass. ``communicator`` (a ``parallel.comm.Communicator``) moves the collectives onto the peer-memory
kernels; otherwise ``torch.distributed`` runs them (gloo in the CPU tests, NCCL on GPUs).

Memory per rank against plain data parallel: gradients numel / world (+ one bucket in flight), optimizer state
numel / world; parameters unchanged. Between "optimizer" (ZeRO-1: ``parallel.dp``) and "parameters" (``parallel.zero3``).

Reference: ShardMode.Gradients (src/Idrak.Network/Training/Sharding.cs:69,184).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn


class _Bucket:
    def __init__(self, params: List[nn.Parameter], world: int, rank: int):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        self.padded = (self.numel + world - 1) // world * world
        self.shard_len = self.padded // world
        p0 = params[0]
        self.dtype, self.device = p0.dtype, p0.device
        flat = torch.zeros(self.padded, dtype=torch.float32, device=self.device)
        off = 0
        self.offsets = []
        for p in params:
            flat[off: off + p.numel()].copy_(p.detach().reshape(-1).float())
            self.offsets.append(off)
            off += p.numel()
        # fp32 master copy of this rank's slice: what the optimizer steps
        self.shard = nn.Parameter(flat[rank * self.shard_len: (rank + 1) * self.shard_len].clone())
        self.waiting = len(params)
        self.work = None
        self.staged: Optional[torch.Tensor] = None
        self.reduced: Optional[torch.Tensor] = None


class ShardedGradients:
    def __init__(self, model: nn.Module, bucket_elems: int = 1 << 22, group=None, communicator=None):
        self.model, self.group, self.comm = model, group, communicator
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        params = [p for p in model.parameters() if p.requires_grad]
        self.buckets: List[_Bucket] = []
        cur: List[nn.Parameter] = []
        size = 0
        for p in reversed(params):
            if cur and (size + p.numel() > bucket_elems or p.dtype != cur[0].dtype or p.device != cur[0].device):
                self.buckets.append(_Bucket(cur, self.world, self.rank))
                cur, size = [], 0
            cur.append(p)
            size += p.numel()
        if cur:
            self.buckets.append(_Bucket(cur, self.world, self.rank))
        self._bucket_of: Dict[int, _Bucket] = {id(p): b for b in self.buckets for p in b.params}
        self.handles = [p.register_post_accumulate_grad_hook(self._on_gradient) for p in params]
        self.peak_full_gradient_elems = 0

    # ------------------------------------------------------------------ backward
    def _on_gradient(self, p: nn.Parameter) -> None:
        b = self._bucket_of[id(p)]
        b.waiting -= 1
        if b.waiting == 0:
            self._reduce(b)

    def _reduce(self, b: _Bucket) -> None:
        live = sum(q.grad.numel() for bb in self.buckets for q in bb.params if q.grad is not None)
        self.peak_full_gradient_elems = max(self.peak_full_gradient_elems, live)
        flat = torch.zeros(b.padded, dtype=torch.float32, device=b.device)
        for p, off in zip(b.params, b.offsets):
            if p.grad is not None:
                flat[off: off + p.numel()].copy_(p.grad.reshape(-1))
                p.grad = None                                  # the full gradient is gone from here on
        mine = torch.empty(b.shard_len, dtype=torch.float32, device=b.device)
        if self.world == 1:
            mine.copy_(flat[: b.shard_len])
        elif self.comm is not None:
            buf = self.comm.symmetric(b.padded * 4)
            buf.tensor(torch.float32, b.padded).copy_(flat)
            self.comm.reduce_scatter(buf, torch.float32, b.padded, mine)
            buf.close()
        else:
            b.staged = flat
            b.work = dist.reduce_scatter_tensor(mine, flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        b.reduced = mine

    def finish_backward(self, weight: Optional[float] = None) -> None:
        """After ``loss.backward()``: waits for the reductions and hands each shard its gradient (the ranks' mean, or
        the sum times ``weight``)."""
        scale = weight if weight is not None else 1.0 / self.world
        for b in self.buckets:
            if b.waiting != 0 and any(p.grad is not None for p in b.params):
                self._reduce(b)                                # a bucket with parameters that got no gradient
            if b.work is not None:
                b.work.wait()
                b.work, b.staged = None, None
            if b.reduced is not None:
                g = b.reduced.mul_(scale)
                b.shard.grad = g if b.shard.grad is None else b.shard.grad.add_(g)
                b.reduced = None
            b.waiting = len(b.params)

    # ------------------------------------------------------------------ after the optimizer step
    def publish(self) -> None:
        """All-gathers the stepped shards and writes them into the parameters (cast to the parameters' dtype)."""
        for b in self.buckets:
            full = torch.empty(b.padded, dtype=torch.float32, device=b.device)
            if self.world > 1:
                dist.all_gather_into_tensor(full, b.shard.detach(), group=self.group)
            else:
                full.copy_(b.shard.detach())
            with torch.no_grad():
                for p, off in zip(b.params, b.offsets):
                    p.copy_(full[off: off + p.numel()].view(p.shape))

    def parameters(self) -> List[nn.Parameter]:
        return [b.shard for b in self.buckets]

    def gradient_elems_held(self) -> int:
        """Gradient elements this rank holds between backward and the optimizer step."""
        full = sum(q.grad.numel() for b in self.buckets for q in b.params if q.grad is not None)
        return full + sum(b.shard.grad.numel() for b in self.buckets if b.shard.grad is not None)

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []
