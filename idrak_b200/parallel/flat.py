"""Flat parameter / gradient storage.

All parameters of a model are moved into one contiguous buffer (and their gradients into another) with
every tensor starting on a 256-byte boundary. One collective or one fused reduce + update kernel then
covers the whole model, and a rank's shard of the optimizer state is a contiguous slice.

Reference: BucketLayout packs (parameter, offset, count) pieces in reverse parameter order
(src/Idrak.Network/Training/GradientBuckets.cs:19-110); here the pieces live in one allocation, and the
bucket boundaries are offsets into it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence

import torch

ALIGN_ELEMS = 128      # 256 bytes of bf16


@dataclass
class Piece:
    index: int         # position in the parameter list
    offset: int        # first element in the flat buffer
    numel: int


class FlatBuffers:
    """Re-homes ``params`` into a flat buffer; ``p.data`` and ``p.grad`` become views of the flat tensors."""

    def __init__(self, params: Iterable[torch.nn.Parameter], grad_dtype: torch.dtype | None = None,
                 allocator=None, reverse: bool = True, pad_to: int = 1):
        self.params = [p for p in params]
        assert self.params, "no parameters"
        dev, dtype = self.params[0].device, self.params[0].dtype
        assert all(p.dtype == dtype and p.device == dev for p in self.params), "mixed dtypes / devices"
        order = list(range(len(self.params)))
        if reverse:
            order.reverse()      # gradients become ready roughly in reverse parameter order
        self.pieces: list[Piece] = []
        off = 0
        for i in order:
            n = self.params[i].numel()
            self.pieces.append(Piece(i, off, n))
            off += (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        self.numel = (off + pad_to - 1) // pad_to * pad_to
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=dev))
        self.param = alloc(self.numel, dtype)
        self.grad = alloc(self.numel, grad_dtype or dtype)
        with torch.no_grad():
            for pc in self.pieces:
                p = self.params[pc.index]
                view = self.param[pc.offset: pc.offset + pc.numel].view_as(p)
                view.copy_(p.data)
                p.data = view
                p.grad = self.grad[pc.offset: pc.offset + pc.numel].view_as(p)

    def piece_of(self, index: int) -> Piece:
        for pc in self.pieces:
            if pc.index == index:
                return pc
        raise KeyError(index)

    def buckets(self, bucket_elems: int) -> list[tuple[int, int, list[int]]]:
        """Split the flat range into buckets of about ``bucket_elems``: (start, end, parameter indices)."""
        out, start, members = [], 0, []
        for pc in self.pieces:
            members.append(pc.index)
            end = pc.offset + (pc.numel + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
            if end - start >= bucket_elems:
                out.append((start, end, members))
                start, members = end, []
        if members or start < self.numel:
            out.append((start, self.numel, members))
        return out

    def zero_grad(self):
        self.grad.zero_()

    def rebind_grads(self):
        """Point ``p.grad`` back at the flat buffer (after something set it to None)."""
        for pc in self.pieces:
            p = self.params[pc.index]
            p.grad = self.grad[pc.offset: pc.offset + pc.numel].view_as(p)
