"""Direct parameter-gradient writes.

PyTorch's autograd hands a weight gradient to an ``AccumulateGrad`` node that adds it into ``p.grad``
with one more kernel and a pass over memory per parameter, after ``zero_grad`` has filled the same
memory with zeros. The fused functions of this package can instead let the kernel that computes a
weight gradient store it straight into ``p.grad`` (``beta = 0`` the first time a parameter is written in
a step, accumulate afterwards) and return ``None`` to autograd.

A parameter opts in with :func:`enable` (its ``.grad`` must already exist, e.g. a view of a flat
buffer). :func:`next_step` starts a new step: the first write of every parameter overwrites again, so
no zero-fill is needed. A parameter whose ``_idrak_ready`` attribute is callable gets it called after
each direct write — the data-parallel bucket logic hangs off that, as it would off the
post-accumulate hook (the reference's per-parameter "gradient ready" notification,
src/Idrak.Abstraction/Tensors/Autograd.cs:146-164).
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch

_EPOCH = 0


def next_step() -> None:
    global _EPOCH
    _EPOCH += 1


def enable(params: Iterable[torch.nn.Parameter]) -> None:
    for p in params:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        p._idrak_direct = True
        p._idrak_epoch = -1


def disable(params: Iterable[torch.nn.Parameter]) -> None:
    for p in params:
        p._idrak_direct = False


def target(param: Optional[torch.Tensor]) -> Optional[Tuple[torch.Tensor, bool]]:
    """(gradient tensor to write, accumulate?) when ``param`` takes direct writes, else None."""
    if param is None or not getattr(param, "_idrak_direct", False) or param.grad is None:
        return None
    accumulate = getattr(param, "_idrak_epoch", -1) == _EPOCH
    param._idrak_epoch = _EPOCH
    return param.grad, accumulate


def written(param: torch.Tensor) -> None:
    """Tell listeners that ``param``'s gradient is complete. A parameter written from several places in one
    backward pass (a table shared by the embedding and the output head) sets ``_idrak_writers`` to that
    number, and the notification goes out after the last of them."""
    writers = getattr(param, "_idrak_writers", 1)
    if writers > 1:
        epoch, count = getattr(param, "_idrak_write_count", (-1, 0))
        count = count + 1 if epoch == _EPOCH else 1
        param._idrak_write_count = (_EPOCH, count)
        if count % writers != 0:
            return
    cb = getattr(param, "_idrak_ready", None)
    if cb is not None:
        cb()
