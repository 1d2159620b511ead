"""Parameter sharding ("parameters" mode of the sharded data parallel): every rank keeps 1 / world of each block's
weights, gathers a block's full weights just before the block runs (forward and again for backward), frees them right
after, and reduce-scatters the block's gradients so each rank ends with the gradient of its own shard. Optimizer state
exists for the shard only. Memory per rank: shards + one or two gathered blocks, instead of the whole model.

    sharded = ShardedParameters(model, units=model.blocks, group=group)     # other parameters stay replicated
    opt = torch.optim.AdamW(sharded.parameters(), lr=...)
    loss = model.loss(ids, targets); loss.backward(); sharded.finish_backward(); opt.step(); opt.zero_grad()

Each unit's parameters live in one flat buffer (padded to a multiple of the world size). The gather is one
``all_gather_into_tensor`` into that buffer; parameters are views of it, and freeing is a storage resize to zero, so
autograd's saved references stay valid objects and see the re-gathered values in backward. Gradients of a unit are
flattened in the unit's backward hook and reduce-scattered (sum, divided by the world size).

Reference: the "parameters" mode of the reference's sharded sync (src/Idrak.Network/Training/Sharding.cs:592-844: master
copies, evict / recompute, forward hooks that gather per module within a byte budget).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import nn


class _Unit:
    def __init__(self, module: nn.Module, group, world: int, rank: int):
        self.module, self.group, self.world, self.rank = module, group, world, rank
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("a sharded unit needs trainable parameters")
        p0 = self.params[0]
        if any(p.dtype != p0.dtype or p.device != p0.device for p in self.params):
            raise ValueError("the parameters of a sharded unit must share dtype and device")
        self.numel = sum(p.numel() for p in self.params)
        self.padded = (self.numel + world - 1) // world * world
        self.shard_len = self.padded // world
        self.full = torch.zeros(self.padded, dtype=p0.dtype, device=p0.device)
        off = 0
        self.slices = []
        for p in self.params:
            self.full[off: off + p.numel()].copy_(p.detach().reshape(-1))
            self.slices.append((off, p.numel(), p.shape))
            off += p.numel()
        # the shard this rank owns: a leaf parameter the optimizer steps
        self.shard = nn.Parameter(self.full[rank * self.shard_len: (rank + 1) * self.shard_len].clone())
        self._bytes = self.full.untyped_storage().nbytes()
        for p, (o, n, shape) in zip(self.params, self.slices):
            p.data = self.full[o: o + n].view(shape)
        self.gathered = True
        self.free()

    # ------------------------------------------------------------------ gather / free
    def gather(self) -> None:
        if self.gathered:
            return
        self.full.untyped_storage().resize_(self._bytes)
        if self.world > 1:
            dist.all_gather_into_tensor(self.full, self.shard.detach(), group=self.group)
        else:
            self.full.copy_(self.shard.detach())
        self.gathered = True

    def free(self) -> None:
        if self.gathered:
            self.full.untyped_storage().resize_(0)
            self.gathered = False

    # ------------------------------------------------------------------ gradients
    def reduce_gradients(self) -> None:
        """Flatten the unit's gradients, reduce-scatter them and accumulate into the shard's gradient."""
        p0 = self.params[0]
        flat = torch.zeros(self.padded, dtype=p0.dtype, device=p0.device)
        any_grad = False
        for p, (o, n, _) in zip(self.params, self.slices):
            if p.grad is not None:
                flat[o: o + n].copy_(p.grad.reshape(-1))
                p.grad = None
                any_grad = True
        if not any_grad and self.world == 1:
            return
        mine = torch.empty(self.shard_len, dtype=p0.dtype, device=p0.device)
        if self.world > 1:
            dist.reduce_scatter_tensor(mine, flat, op=dist.ReduceOp.SUM, group=self.group)
            mine.div_(self.world)
        else:
            mine.copy_(flat[: self.shard_len])
        if self.shard.grad is None:
            self.shard.grad = mine
        else:
            self.shard.grad.add_(mine)


class ShardedParameters:
    def __init__(self, model: nn.Module, units: Optional[Sequence[nn.Module]] = None, group=None):
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        units = list(units) if units is not None else [m for m in model.children() if any(p.requires_grad for p in m.parameters())]
        self.units = [_Unit(m, group, self.world, self.rank) for m in units]
        unit_params = {id(p) for u in self.units for p in u.params}
        self.replicated = [p for p in model.parameters() if p.requires_grad and id(p) not in unit_params]
        self._pending: List[_Unit] = []
        self.handles = []
        for u in self.units:
            self.handles.append(u.module.register_forward_pre_hook(lambda m, a, u=u: u.gather()))
            self.handles.append(u.module.register_forward_hook(lambda m, a, o, u=u: self._after_forward(u)))
            self.handles.append(u.module.register_full_backward_pre_hook(lambda m, g, u=u: u.gather()))
            self.handles.append(u.module.register_full_backward_hook(lambda m, gi, go, u=u: self._after_backward(u)))

    def _after_forward(self, u: _Unit) -> None:
        u.free()

    def _after_backward(self, u: _Unit) -> None:
        # parameter gradients of the unit are accumulated after this hook returns (they belong to the same backward
        # node group): reduce them at the next unit's hook or in finish_backward
        self._flush()
        self._pending.append(u)

    def _flush(self) -> None:
        for u in self._pending:
            u.reduce_gradients()
            u.free()
        self._pending = []

    def finish_backward(self) -> None:
        """Call after ``loss.backward()``: reduces what is still pending and averages the replicated parameters' gradients."""
        self._flush()
        for u in self.units:                       # units whose inputs needed no gradient never saw a backward hook
            if any(p.grad is not None for p in u.params):
                u.reduce_gradients()
            u.free()
        if self.world > 1:
            for p in self.replicated:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.group)
                    p.grad.div_(self.world)

    def parameters(self) -> List[nn.Parameter]:
        """What the optimizer steps: this rank's shards plus the replicated parameters."""
        return [u.shard for u in self.units] + self.replicated

    def gathered_bytes(self) -> int:
        return sum(u.full.untyped_storage().nbytes() for u in self.units)

    def full_state(self) -> dict:
        """The whole model's parameters (gathered on every rank) by name, e.g. for a checkpoint."""
        for u in self.units:
            u.gather()
        state = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        for u in self.units:
            u.free()
        return state

    def remove(self) -> None:
        """Gather everything back and detach the hooks (the model becomes an ordinary replicated model again)."""
        for h in self.handles:
            h.remove()
        self.handles = []
        for u in self.units:
            u.gather()
            for p, (o, n, shape) in zip(u.params, u.slices):
                p.data = u.full[o: o + n].view(shape).clone()
