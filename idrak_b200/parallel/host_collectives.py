"""Collectives over host values built from point-to-point messages, with the algorithm as a registered choice:
``naive`` (everything to the first rank, summed in rank order, sent back), ``ring`` (reduce-scatter then all-gather:
2 (W − 1) / W of the values leave each rank, fixed order of additions, chain broadcast) and ``hierarchical`` (sum inside
each node, one ring per column across nodes, spread inside each node; nodes may differ in size).

    coll = create("ring", TorchTransport())                 # ranks of torch.distributed (gloo or nccl process group)
    coll = create("hierarchical", SimRankTransport(ctx), nodes=[[0, 1, 2], [3, 4]])
    total = coll.all_reduce(values)                          # identical bits on every rank
    mine = coll.reduce_scatter(values, counts)               # uneven pieces
    whole = coll.all_gather(mine, counts)
    got = coll.all_to_all(pieces)                            # one piece per peer, pairwise rounds

Values are float32 on the host; ``wire="bfloat16"`` halves the bytes of every message (values are rounded once per
hop). The fused peer-memory kernels of ``parallel.dp`` / ``parallel.comm`` are the fast path on one NVLink box; these
serve control values, CPU ranks, the cluster simulator and anything that crosses nodes without NCCL.

Reference: src/Idrak.Network/Collectives/Algorithms.cs:15-201 (naive, ring), HierarchicalCollectives.cs:27 (column
plan for uneven nodes), Abstractions/HostCollectives.cs:454-493,654-753 (pairwise all-to-all, uneven pieces, the
chunk-interleaved exchange that keeps rings from deadlocking), WireValues.cs:14 (f32 / bf16 wire encodings).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch


# ------------------------------------------------------------------------------------------------ transports
class Transport:
    """Point-to-point messages of float32 / bfloat16 vectors between numbered ranks."""

    rank: int
    world: int

    def exchange(self, dst: Optional[int], out: Optional[torch.Tensor], src: Optional[int], count: int,
                 dtype: torch.dtype) -> Optional[torch.Tensor]:
        """Send ``out`` to ``dst`` and receive ``count`` values from ``src`` at the same time (either side may be None)."""
        raise NotImplementedError


class TorchTransport(Transport):
    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def _global(self, r: int) -> int:
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def exchange(self, dst, out, src, count, dtype):
        work = self.dist.isend(out.contiguous(), self._global(dst), group=self.group) if dst is not None else None
        got = None
        if src is not None:
            got = torch.empty(count, dtype=dtype)
            self.dist.recv(got, self._global(src), group=self.group)
        if work is not None:
            work.wait()
        return got


class SimRankTransport(Transport):
    """The cluster simulator's rank context as a transport (its sends never block, so exchange is send then receive)."""

    def __init__(self, ctx):
        self.ctx, self.rank, self.world = ctx, ctx.rank, ctx.world

    def exchange(self, dst, out, src, count, dtype):
        if dst is not None:
            self.ctx.send(dst, out.clone(), out.numel() * out.element_size())
        return self.ctx.recv(src, "collective piece") if src is not None else None


# ------------------------------------------------------------------------------------------------ base
def even_counts(n: int, parts: int) -> List[int]:
    base, extra = divmod(n, parts)
    return [base + (1 if i < extra else 0) for i in range(parts)]


class HostCollectives:
    name = "?"

    def __init__(self, transport: Transport, wire: str = "float32", chunk: int = 1 << 20):
        if wire not in ("float32", "bfloat16"):
            raise ValueError("wire must be 'float32' or 'bfloat16'")
        self.t, self.rank, self.world = transport, transport.rank, transport.world
        self.wire = torch.float32 if wire == "float32" else torch.bfloat16
        self.chunk = int(chunk)                       # values per message: long vectors go as several exchanges
        self.bytes_sent = 0
        self.messages = 0

    # one hop, chunked so that no message is larger than ``chunk`` values
    def _swap(self, dst, out: Optional[torch.Tensor], src, count: int) -> Optional[torch.Tensor]:
        n_out = out.numel() if out is not None else 0
        pieces = []
        steps = max(-(-n_out // self.chunk) if dst is not None else 0, -(-count // self.chunk) if src is not None else 0, 1)
        for i in range(steps):
            lo_o, hi_o = min(i * self.chunk, n_out), min((i + 1) * self.chunk, n_out)
            lo_i, hi_i = min(i * self.chunk, count), min((i + 1) * self.chunk, count)
            send = dst is not None and hi_o > lo_o            # empty pieces are not sent: both ends know the sizes
            recv = src is not None and hi_i > lo_i
            o = out[lo_o:hi_o].to(self.wire) if send else None
            if send:
                self.bytes_sent += o.numel() * o.element_size()
                self.messages += 1
            got = self.t.exchange(dst if send else None, o, src if recv else None, hi_i - lo_i, self.wire)
            if recv:
                pieces.append(got.float())
        if src is None:
            return None
        if not pieces:
            return torch.zeros(0)
        return torch.cat(pieces) if len(pieces) != 1 else pieces[0]

    def _send(self, dst, out):
        self._swap(dst, out, None, 0)

    def _recv(self, src, count):
        return self._swap(None, None, src, count)

    # ---- ring pieces over an ordered list of ranks (this rank must be in it)
    def _ring_reduce_scatter(self, ranks: Sequence[int], v: torch.Tensor, counts: Sequence[int]) -> None:
        """After this, piece ``i`` of ``v`` on ``ranks[i]`` holds the sum over ``ranks`` (other pieces hold partial sums)."""
        w = len(ranks)
        if w == 1:
            return
        me = ranks.index(self.rank)
        offs = [0]
        for c in counts:
            offs.append(offs[-1] + c)
        right, left = ranks[(me + 1) % w], ranks[(me - 1) % w]
        for s in range(w - 1):
            ps, pr = (me - s - 1) % w, (me - s - 2) % w
            got = self._swap(right, v[offs[ps]:offs[ps + 1]], left, counts[pr])
            v[offs[pr]:offs[pr + 1]] += got

    def _ring_all_gather(self, ranks: Sequence[int], v: torch.Tensor, counts: Sequence[int]) -> None:
        """Piece ``i`` of ``v`` is valid on ``ranks[i]``; afterwards every piece is valid everywhere in ``ranks``."""
        w = len(ranks)
        if w == 1:
            return
        me = ranks.index(self.rank)
        offs = [0]
        for c in counts:
            offs.append(offs[-1] + c)
        right, left = ranks[(me + 1) % w], ranks[(me - 1) % w]
        for s in range(w - 1):
            ps, pr = (me - s) % w, (me - s - 1) % w
            v[offs[pr]:offs[pr + 1]] = self._swap(right, v[offs[ps]:offs[ps + 1]], left, counts[pr])

    # ---- the public calls; algorithms override all_reduce / broadcast
    def all_reduce(self, values: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def broadcast(self, values: torch.Tensor, root: int = 0) -> torch.Tensor:
        v = values.detach().float().reshape(-1)
        if self.rank == root:
            for r in range(self.world):
                if r != root:
                    self._send(r, v)
            return (v.to(self.wire).float() if self.wire != torch.float32 else v.clone()).reshape(values.shape)
        return self._recv(root, v.numel()).reshape(values.shape)

    def reduce_scatter(self, values: torch.Tensor, counts: Optional[Sequence[int]] = None) -> torch.Tensor:
        """This rank's piece of the sum; ``counts[i]`` values belong to rank ``i`` (default: as even as possible)."""
        v = values.detach().float().reshape(-1).clone()
        counts = list(counts) if counts is not None else even_counts(v.numel(), self.world)
        if sum(counts) != v.numel() or len(counts) != self.world:
            raise ValueError("counts must have one entry per rank and add up to the number of values")
        ranks = list(range(self.world))
        # the ring leaves piece (me + 1) complete on rank me, so run it over pieces shifted by one
        self._ring_reduce_scatter(ranks, v, counts)
        off = sum(counts[: self.rank])
        return v[off: off + counts[self.rank]].clone()

    def all_gather(self, piece: torch.Tensor, counts: Optional[Sequence[int]] = None) -> torch.Tensor:
        p = piece.detach().float().reshape(-1)
        counts = list(counts) if counts is not None else [p.numel()] * self.world
        if counts[self.rank] != p.numel():
            raise ValueError("this rank's piece does not have the announced size")
        v = torch.zeros(sum(counts))
        off = sum(counts[: self.rank])
        v[off: off + p.numel()] = p.to(self.wire).float() if self.wire != torch.float32 else p
        self._ring_all_gather(list(range(self.world)), v, counts)
        return v

    def all_to_all(self, pieces: Sequence[torch.Tensor], counts_in: Optional[Sequence[int]] = None) -> List[torch.Tensor]:
        """``pieces[j]`` goes to rank ``j``; returns what every rank sent here. W − 1 pairwise rounds."""
        if len(pieces) != self.world:
            raise ValueError("one piece per rank")
        if counts_in is None:                          # sizes travel first, as one small all-to-all of their own
            sizes = [torch.tensor([float(p.numel())]) for p in pieces]
            counts_in = [int(x.item()) for x in self.all_to_all(sizes, [1] * self.world)]
        own = pieces[self.rank].detach().float().reshape(-1)
        out: List[Optional[torch.Tensor]] = [None] * self.world
        out[self.rank] = own.to(self.wire).float() if self.wire != torch.float32 else own.clone()
        for s in range(1, self.world):
            dst, src = (self.rank + s) % self.world, (self.rank - s) % self.world
            out[src] = self._swap(dst, pieces[dst].detach().float().reshape(-1), src, counts_in[src])
        return out  # type: ignore[return-value]

    def barrier(self) -> None:
        self.all_reduce(torch.zeros(1))


# ------------------------------------------------------------------------------------------------ algorithms
class NaiveCollectives(HostCollectives):
    name = "naive"

    def all_reduce(self, values):
        v = values.detach().float().reshape(-1).clone()
        if self.world == 1:
            return v.reshape(values.shape)
        if self.rank == 0:
            for r in range(1, self.world):            # rank order: the same additions whatever arrives first
                v += self._recv(r, v.numel())
            for r in range(1, self.world):
                self._send(r, v)
            if self.wire != torch.float32:
                v = v.to(self.wire).float()
            return v.reshape(values.shape)
        self._send(0, v)
        return self._recv(0, v.numel()).reshape(values.shape)


class RingCollectives(HostCollectives):
    name = "ring"

    def all_reduce(self, values):
        v = values.detach().float().reshape(-1).clone()
        ranks = list(range(self.world))
        counts = even_counts(v.numel(), self.world)
        self._ring_reduce_scatter(ranks, v, counts)
        if self.wire != torch.float32:                 # the owner's piece takes the same rounding its copies will
            off = sum(counts[: self.rank])
            v[off: off + counts[self.rank]] = v[off: off + counts[self.rank]].to(self.wire).float()
        self._ring_all_gather(ranks, v, counts)
        return v.reshape(values.shape)

    def broadcast(self, values, root=0):
        """Chain: each rank passes the values on to the next, so the root sends them once."""
        v = values.detach().float().reshape(-1)
        order = [(root + i) % self.world for i in range(self.world)]
        at = order.index(self.rank)
        if at > 0:
            v = self._recv(order[at - 1], v.numel())
        elif self.wire != torch.float32:
            v = v.to(self.wire).float()
        if at + 1 < self.world:
            self._send(order[at + 1], v)
        return v.clone().reshape(values.shape)


class HierarchicalCollectives(RingCollectives):
    """``nodes``: the ranks of each node. The number of columns is the size of the smallest node; in a larger node the
    ranks beyond that first hand their values to a column rank of their node and get the result from it at the end."""

    name = "hierarchical"

    def __init__(self, transport, nodes: Sequence[Sequence[int]], **kw):
        super().__init__(transport, **kw)
        self.nodes = [list(n) for n in nodes]
        flat = sorted(r for n in self.nodes for r in n)
        if flat != list(range(self.world)) or any(not n for n in self.nodes):
            raise ValueError("nodes must list every rank exactly once and no node may be empty")
        self.columns = min(len(n) for n in self.nodes)
        self.node = next(n for n in self.nodes if self.rank in n)
        self.local = self.node.index(self.rank)

    def all_reduce(self, values):
        v = values.detach().float().reshape(-1).clone()
        c = self.columns
        heads, extras = self.node[:c], self.node[c:]
        if self.local >= c:                            # an extra rank: hand over, then wait for the result
            keeper = heads[self.local % c]
            self._send(keeper, v)
            return self._recv(keeper, v.numel()).reshape(values.shape)
        mine = [r for i, r in enumerate(extras) if (c + i) % c == self.local]
        for r in mine:                                 # in rank order
            v += self._recv(r, v.numel())
        counts = even_counts(v.numel(), c)
        self._ring_reduce_scatter(heads, v, counts)    # piece `local` of the node's sum is now complete here
        off = sum(counts[: self.local])
        piece = v[off: off + counts[self.local]].clone()
        column = [n[self.local] for n in self.nodes]   # the same column of every node
        sub = even_counts(piece.numel(), len(column))
        self._ring_reduce_scatter(column, piece, sub)
        if self.wire != torch.float32:
            at = column.index(self.rank)
            o = sum(sub[:at])
            piece[o: o + sub[at]] = piece[o: o + sub[at]].to(self.wire).float()
        self._ring_all_gather(column, piece, sub)
        v[off: off + counts[self.local]] = piece
        self._ring_all_gather(heads, v, counts)
        for r in mine:
            self._send(r, v)
        return v.reshape(values.shape)


COLLECTIVES: Dict[str, Callable[..., HostCollectives]] = {
    "naive": NaiveCollectives, "ring": RingCollectives, "hierarchical": HierarchicalCollectives}


def create(name: str, transport: Transport, **options) -> HostCollectives:
    if name not in COLLECTIVES:
        raise KeyError(f"Collective algorithm '{name}' is not registered. Known: {', '.join(sorted(COLLECTIVES))}")
    return COLLECTIVES[name](transport, **options)
