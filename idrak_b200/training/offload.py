"""Keeping state off the GPU: a host optimizer (moments and the update on the CPU, gradients staged through pinned
memory), layer-scoped weight offloading with prefetch, and parameter groups over several optimizers.

* ``HostOptimizer`` - AdamW whose fp32 master weights and moments live in pinned host memory. A step copies each
  gradient to its pinned slot on a side stream (overlapping the rest of the copies), updates on the CPU, and copies
  the new weights back. The GPU holds only bf16 weights and gradients: 4 bytes per parameter instead of 16.
* ``LayerOffloader`` - weights of a stack of blocks parked in pinned host memory; a forward pre-hook brings block
  ``i`` in (and starts block ``i + 1``'s copy on a side stream), a forward hook sends block ``i`` back out. ``resident``
  blocks stay on the GPU; the coldest-first policy keeps the first blocks in while later ones stream.
* ``GroupedOptimizer`` - several optimizers, each over its own parameters, stepped and saved as one.

Reference: HostOptimizer (src/Idrak/Optimizers/HostOptimizer.cs:19-395: pinned staged gradient download,
IHostGradients), Offloading (src/Idrak/Offloading.cs: layer-scoped staging, prefetch, cold-first), GroupedOptimizer.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Sequence

import torch
from torch import nn


def _pinned_like(t: torch.Tensor, dtype=None) -> torch.Tensor:
    out = torch.empty(t.shape, dtype=dtype or t.dtype, device="cpu")
    return out.pin_memory() if torch.cuda.is_available() else out


class HostOptimizer:
    def __init__(self, params: Iterable, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.0):
        groups = list(params)
        if groups and not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        self.param_groups = [{"lr": lr, "weight_decay": weight_decay, **g, "params": list(g["params"])} for g in groups]
        self.params: List[torch.nn.Parameter] = [p for g in self.param_groups for p in g["params"]]
        self._wd = [g["weight_decay"] for g in self.param_groups for _ in g["params"]]
        self._lr_scale = [g["lr"] / lr if lr else 1.0 for g in self.param_groups for _ in g["params"]]
        self.lr, self.betas, self.eps, self.max_grad_norm = lr, betas, eps, max_grad_norm
        self.step_count = 0
        self.master = [_pinned_like(p, torch.float32).copy_(p.detach().float()) for p in self.params]
        self.m = [torch.zeros_like(w) for w in self.master]
        self.v = [torch.zeros_like(w) for w in self.master]
        self.staged = [_pinned_like(p, torch.float32 if not p.is_cuda else p.dtype) for p in self.params]
        self.copy_stream = torch.cuda.Stream() if any(p.is_cuda for p in self.params) else None
        self.last_grad_norm = 0.0

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def step(self) -> float:
        """Download gradients, clip by the global norm, update on the host, upload the weights. Returns the norm."""
        live = [i for i, p in enumerate(self.params) if p.grad is not None]
        if self.copy_stream is not None:
            self.copy_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.copy_stream):
                for i in live:
                    self.staged[i].copy_(self.params[i].grad, non_blocking=True)
            self.copy_stream.synchronize()
        else:
            for i in live:
                self.staged[i].copy_(self.params[i].grad)
        grads = {i: self.staged[i].float() for i in live}
        norm = math.sqrt(sum(float(g.pow(2).sum()) for g in grads.values()))
        self.last_grad_norm = norm
        if not math.isfinite(norm):
            return norm                                   # a step with overflowed gradients is skipped
        clip = min(1.0, self.max_grad_norm / (norm + 1e-6)) if self.max_grad_norm > 0 else 1.0
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        for i in live:
            g = grads[i] * clip
            lr = self.lr * self._lr_scale[i]
            w, m, v = self.master[i], self.m[i], self.v[i]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            if self._wd[i]:
                w.mul_(1 - lr * self._wd[i])
            w.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-lr)
            self.params[i].data.copy_(w, non_blocking=True)
        return norm

    def state_dict(self) -> Dict[str, torch.Tensor]:
        out = {"step": torch.tensor(self.step_count)}
        for i in range(len(self.params)):
            out[f"m.{i}"], out[f"v.{i}"], out[f"master.{i}"] = self.m[i].clone(), self.v[i].clone(), self.master[i].clone()
        return out

    def load_state_dict(self, state: Dict[str, torch.Tensor]) -> None:
        self.step_count = int(state["step"])
        for i in range(len(self.params)):
            self.m[i].copy_(state[f"m.{i}"])
            self.v[i].copy_(state[f"v.{i}"])
            if f"master.{i}" in state:
                self.master[i].copy_(state[f"master.{i}"])
                self.params[i].data.copy_(self.master[i])


class GroupedOptimizer:
    """``GroupedOptimizer({"body": opt_a, "head": opt_b})``: one ``step`` / ``zero_grad`` / state for all of them."""

    def __init__(self, optimizers: Dict[str, object]):
        self.optimizers = dict(optimizers)
        seen = set()
        for name, o in self.optimizers.items():
            for p in _params_of(o):
                if id(p) in seen:
                    raise ValueError(f"a parameter appears in more than one group (found again in '{name}')")
                seen.add(id(p))

    def step(self):
        return {name: o.step() for name, o in self.optimizers.items()}

    def zero_grad(self, set_to_none: bool = True):
        for o in self.optimizers.values():
            o.zero_grad(set_to_none)

    def state_dict(self):
        return {name: o.state_dict() for name, o in self.optimizers.items()}

    def load_state_dict(self, state):
        for name, o in self.optimizers.items():
            if name not in state:
                raise KeyError(f"the saved state has no group '{name}'; groups: {', '.join(state)}")
            o.load_state_dict(state[name])


def _params_of(o) -> List:
    if hasattr(o, "params"):
        return list(o.params)
    return [p for g in o.param_groups for p in g["params"]]


# ---------------------------------------------------------------------------------------------------------------------
class LayerOffloader:
    """Stream a stack of blocks through the GPU.

        off = LayerOffloader(model.blocks, device="cuda", resident=4)     # first 4 blocks stay in; the rest stream
        y = model(x)                                                       # hooks move weights around the forward
        off.remove()

    Host copies are pinned; block ``i + 1`` is fetched on a side stream while block ``i`` computes. Intended for
    inference and for frozen bases (weights that change on the GPU are not written back)."""

    def __init__(self, blocks: Sequence[nn.Module], device="cuda", resident: int = 0, prefetch: bool = True):
        self.blocks = list(blocks)
        self.device = torch.device(device)
        self.resident, self.prefetch = resident, prefetch
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.host: List[Dict[str, torch.Tensor]] = []
        self.ready: Dict[int, Optional[torch.cuda.Event]] = {}
        self.handles = []
        self.fetches = 0
        for i, b in enumerate(self.blocks):
            keep = {}
            for name, p in list(b.named_parameters()) + list(b.named_buffers()):
                keep[name] = _pinned_like(p.detach()).copy_(p.detach()) if self.device.type == "cuda" else p.detach().clone()
            self.host.append(keep)
            if i < resident:
                self._place(i, self.device)
            else:
                self._evict(i)
            self.handles.append(b.register_forward_pre_hook(lambda m, a, i=i: self._before(i)))
            self.handles.append(b.register_forward_hook(lambda m, a, o, i=i: self._after(i)))

    def _tensors(self, i):
        b = self.blocks[i]
        return list(b.named_parameters()) + list(b.named_buffers())

    def _place(self, i: int, device) -> None:
        for name, p in self._tensors(i):
            p.data = self.host[i][name].to(device, non_blocking=True)

    def _evict(self, i: int) -> None:
        for name, p in self._tensors(i):
            p.data = self.host[i][name]                     # the pinned host copy stands in while the block is out

    def _fetch(self, i: int) -> None:
        if i >= len(self.blocks) or i < self.resident or i in self.ready:
            return
        self.fetches += 1
        if self.stream is None:
            self._place(i, self.device)
            self.ready[i] = None
            return
        with torch.cuda.stream(self.stream):
            self._place(i, self.device)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.ready[i] = ev

    def _before(self, i: int) -> None:
        if i < self.resident:
            return
        self._fetch(i)
        ev = self.ready.get(i)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        if self.prefetch:
            self._fetch(i + 1)

    def _after(self, i: int) -> None:
        if i < self.resident:
            return
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())     # the block's kernels finish before its memory is reused
            for _, p in self._tensors(i):
                p.data.record_stream(torch.cuda.current_stream())
        self._evict(i)
        self.ready.pop(i, None)

    def remove(self, to_device: bool = True) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []
        if to_device:
            for i in range(len(self.blocks)):
                self._place(i, self.device)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
