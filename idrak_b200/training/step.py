"""One training step as an object: stage the batch from pinned host memory, forward, backward
(overlapped with gradient reduction when data-parallel), clip + optimizer update, and hand back the
loss. ``Trainer`` drives this; benchmarks and custom loops can use it directly.

With ``use_graph=True`` the device work of a step (forward, backward, update) is recorded once into a
CUDA graph and replayed, which removes the per-kernel launch cost from the host side
(the reference records its fine-tuning step the same way: src/Idrak.Text/FineTuning.cs:3103-3145).

Reference: the loop of samples/Idrak.Samples.GptTraining/Program.cs:296-330 and Trainer.Fit
(src/Idrak/Training/Trainer.cs:400-560).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..ops import _grad


class TrainStep:
    def __init__(self, model: torch.nn.Module, optimizer, *, sync=None, grad_accumulation: int = 1,
                 use_graph: bool = False, loss_fn: Optional[Callable] = None, ignore_index: Optional[int] = None,
                 direct_grads: bool = True):
        self.model, self.optimizer, self.sync = model, optimizer, sync
        self.grad_accumulation = max(1, grad_accumulation)
        self.use_graph = use_graph
        self.loss_fn = loss_fn
        self.ignore_index = ignore_index
        self.device = next(model.parameters()).device
        self._graph = None
        self._static = None
        self._loss_out = None
        self._warm = 0
        self._h2d = None
        self._micro = 0
        self._first_replay = False
        self.graph_kernels = 0
        self.replays = 0
        self._direct = bool(direct_grads) and self.device.type == "cuda"
        self._needs_zero = None
        if self._direct:
            _grad.enable(p for p in model.parameters() if p.requires_grad)
            _grad.next_step()

    # ------------------------------------------------------------------ host -> device staging
    def stage(self, ids_host: torch.Tensor, targets_host: torch.Tensor):
        """Copy a batch that lives in (ideally pinned) host memory into the step's device buffers."""
        if self._static is None or self._static[0].shape != ids_host.shape:
            self._static = (torch.empty(ids_host.shape, dtype=torch.int32, device=self.device),
                            torch.empty(targets_host.shape, dtype=torch.int32, device=self.device))
            self._graph = None
        self._static[0].copy_(ids_host, non_blocking=True)
        self._static[1].copy_(targets_host, non_blocking=True)
        return self._static

    # ------------------------------------------------------------------ the step
    def _loss(self, ids, targets):
        if self.loss_fn is not None:
            return self.loss_fn(self.model, ids, targets)
        return self.model.loss(ids, targets, ignore_index=self.ignore_index)

    def _fwd_bwd(self, ids, targets, last: bool):
        loss = self._loss(ids, targets)
        scaled = loss / self.grad_accumulation if self.grad_accumulation > 1 else loss
        if self.sync is not None and last:
            with self.sync.overlap():
                scaled.backward()
        else:
            scaled.backward()
        return loss.detach()

    def _update(self):
        if self.sync is not None:
            self.sync.reduce_and_step()
        else:
            self.optimizer.step()

    def _eager(self, ids, targets):
        self._micro += 1
        last = self._micro % self.grad_accumulation == 0
        loss = self._fwd_bwd(ids, targets, last)
        if last:
            self._update()
            self._zero_grads()
        return loss

    def _zero_grads(self):
        if self._direct:
            # parameters whose gradient kernels store into .grad need no zero-fill: the first write of the next
            # step overwrites. The rest (gradients that arrive through autograd's accumulate nodes) are zeroed.
            if self._needs_zero is None:
                self._needs_zero = [p for p in self.model.parameters()
                                    if p.grad is not None and getattr(p, "_idrak_epoch", -1) != _grad._EPOCH]
            for p in self._needs_zero:
                p.grad.zero_()
            _grad.next_step()
            return
        if getattr(self.optimizer, "zero_grad_in_step", False):
            return
        if self.sync is not None and hasattr(self.sync, "zero_grad"):
            self.sync.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=False)

    def __call__(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Run one (micro-)step on device tensors; returns the loss as a device scalar."""
        if not self.use_graph or self.grad_accumulation > 1 or not ids.is_cuda:
            return self._eager(ids, targets)
        if self._static is None or self._static[0].data_ptr() != ids.data_ptr():
            if self._static is None or self._static[0].shape != ids.shape:
                self._static = (torch.empty_like(ids, dtype=torch.int32), torch.empty_like(targets, dtype=torch.int32))
                self._graph = None
            self._static[0].copy_(ids)
            self._static[1].copy_(targets)
        if self._graph is None:
            if self._warm < 2:          # eager steps first: lazy state (grads, tables, scratch) gets created
                self._warm += 1
                return self._eager(*self._static)
            self._capture()
            self._first_replay = True
        if not self._first_replay and hasattr(self.optimizer, "advance_for_replay"):
            self.optimizer.advance_for_replay()
        self._first_replay = False
        self.replays += 1
        self._graph.replay()
        return self._loss_out

    def _capture(self):
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        from .. import _native
        before = _native.lib().idrak_launch_count()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                self._loss_out = self._eager(*self._static)
        torch.cuda.current_stream().wait_stream(side)
        self._graph = g
        self.graph_kernels = int(_native.lib().idrak_launch_count() - before)   # this library's kernels per replay
        self.replays = 0

    def step_from_host(self, ids_host: torch.Tensor, targets_host: torch.Tensor) -> float:
        """The end-to-end call: host batch in, python float loss out (one device->host read)."""
        ids, targets = self.stage(ids_host, targets_host)
        loss = self(ids, targets)
        return float(loss.item())
