"""Autograd helpers with the reference's names over PyTorch's tape: no-grad scopes, user functions, and the
gradient-ready hook that data parallelism hangs its bucket reductions on.

Reference: Autograd (src/Idrak.Abstraction/Tensors/Autograd.cs:7-199: NoGrad, Function, OnGradientReady fired per
parameter right after its last reader ran - :146-164) and DifferentiableFunction.cs:21.
"""
from __future__ import annotations

from typing import Callable, Iterable, List

import torch

no_grad = torch.no_grad
enable_grad = torch.enable_grad
Function = torch.autograd.Function


class GradientReadyHandle:
    def __init__(self, handles: List):
        self._handles = handles

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()


def on_gradient_ready(parameters: Iterable[torch.nn.Parameter], fn: Callable[[torch.nn.Parameter], None]) -> GradientReadyHandle:
    """Call ``fn(parameter)`` during backward as soon as that parameter's gradient is final (after accumulation
    into ``.grad``), i.e. before the rest of the backward pass has run - the point where a bucket can start
    reducing. Returns a handle whose ``remove()`` detaches the hooks."""
    handles = []
    for p in parameters:
        if p.requires_grad:
            handles.append(p.register_post_accumulate_grad_hook(fn))
    return GradientReadyHandle(handles)


def backward(loss: torch.Tensor, retain_graph: bool = False) -> None:
    loss.backward(retain_graph=retain_graph)


def gradient_norm(parameters: Iterable[torch.nn.Parameter]) -> torch.Tensor:
    """Global L2 norm of the gradients (fp32, on the gradients' device)."""
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.zeros(())
    return torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float()) for g in grads]))
