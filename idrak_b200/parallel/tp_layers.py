"""A decoder under tensor parallelism with sequence-sharded activations.

``TPDecoder.from_decoder(model, tp)`` slices an ordinary ``Decoder`` for this rank: attention heads and MLP
columns are split across the ranks, the vocabulary (embedding and head) is split by rows, norms are replicated.
Between layers an activation is this rank's block of rows (tokens) ``[M / world, dim]``; the column-parallel
projections gather it inside the GEMM kernel and the row-parallel ones scatter their partial sums back
(``parallel/tp.py``). The cross-entropy works on vocabulary shards: row maxima, sums of exponentials and target
logits are all-reduced, the full logits never exist on one GPU.

Gradients of replicated parameters (norm weights, row-parallel biases) are summed over the ranks by
``sync_replicated_grads`` after backward; ``TPOptimizer`` clips with the global norm over all shards.

The reference trains data-parallel and pipelined only (src/Idrak.Network/Training/*); the block being sharded here
is its decoder block (src/Idrak/Generation/DecoderBlock.cs) and TokenCrossEntropy (src/Idrak/Losses/TokenCrossEntropy.cs).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..models.decoder import Decoder, Norm
from ..models.spec import DecoderSpec
from ..ops.gemm import bias_grad, weight_grad
from .tp import TensorParallel


class _ColumnParallel(torch.autograd.Function):
    """y[M, N_local] = all_gather(x_local) @ W_local^T + b_local."""

    @staticmethod
    def forward(ctx, x_local, weight, bias, tp: TensorParallel):
        y = tp.ag_gemm(x_local, weight, bias=bias)
        ctx.save_for_backward(x_local, weight)
        ctx.tp, ctx.params, ctx.has_bias = tp, (weight, bias), bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_local, weight = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx = tp.gemm_rs(dy, weight, w_mn=True) if ctx.needs_input_grad[0] else None      # dy @ W, rows scattered
        dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy, tp.all_gather_rows(x_local), ctx.params[0])
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = bias_grad(dy, ctx.params[1])
        return dx, dw, db, None


class _RowParallel(torch.autograd.Function):
    """y_local[M / world, N] = rows of sum_ranks(x @ W_local^T) + b + residual_local."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, tp: TensorParallel):
        y = tp.gemm_rs(x, weight, bias=bias, residual=residual)
        ctx.save_for_backward(x, weight)
        ctx.tp, ctx.params = tp, (weight, bias)
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_local):
        x, weight = ctx.saved_tensors
        tp = ctx.tp
        dy_local = dy_local.contiguous()
        dx = tp.ag_gemm(dy_local, weight, w_mn=True) if ctx.needs_input_grad[0] else None   # gather(dy) @ W_local
        dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(tp.all_gather_rows(dy_local), x, ctx.params[0])
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = bias_grad(dy_local, ctx.params[1])        # this rank's rows; summed over ranks with the replicated grads
        dres = dy_local if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None


def column_parallel_linear(x_local, weight, bias, tp):
    return _ColumnParallel.apply(x_local, weight, bias, tp)


def row_parallel_linear(x, weight, bias, residual, tp):
    return _RowParallel.apply(x, weight, bias, residual, tp)


class _VocabParallelEmbedding(torch.autograd.Function):
    """Rows of this rank of the embedded tokens: each rank looks up the ids that fall in its vocabulary shard
    (zeros elsewhere) and the partial results are reduce-scattered."""

    @staticmethod
    def forward(ctx, ids_flat, table, first, tp: TensorParallel):
        local = ids_flat.long() - first
        inside = (local >= 0) & (local < table.shape[0])
        part = table[local.clamp(0, table.shape[0] - 1)] * inside[:, None].to(table.dtype)
        ctx.save_for_backward(local, inside)
        ctx.tp, ctx.rows = tp, table.shape[0]
        return tp.reduce_scatter_rows(part)

    @staticmethod
    def backward(ctx, d_local):
        local, inside = ctx.saved_tensors
        d_full = ctx.tp.all_gather_rows(d_local.contiguous())
        g = torch.zeros(ctx.rows, d_full.shape[1], dtype=torch.float32, device=d_full.device)
        g.index_add_(0, local[inside], d_full[inside].float())
        return None, g.to(d_local.dtype), None, None


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Mean token cross-entropy over logits whose columns are split across the ranks."""

    @staticmethod
    def forward(ctx, logits, targets, first, vocab_local, group):
        x = logits[:, :vocab_local].float()
        m = x.max(-1).values
        if group is not None or dist.is_initialized():
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(x - m[:, None])
        s = e.sum(-1)
        local_t = targets.long() - first
        inside = (local_t >= 0) & (local_t < vocab_local)
        t_logit = torch.where(inside, x.gather(1, local_t.clamp(0, vocab_local - 1)[:, None])[:, 0], torch.zeros_like(m))
        stats = torch.stack([s, t_logit])
        if group is not None or dist.is_initialized():
            dist.all_reduce(stats, group=group)
        s, t_logit = stats[0], stats[1]
        loss = (torch.log(s) + m - t_logit).mean()
        ctx.save_for_backward(e, s, local_t, inside)
        ctx.shape, ctx.dtype, ctx.vocab_local = logits.shape, logits.dtype, vocab_local
        return loss

    @staticmethod
    def backward(ctx, d_loss):
        e, s, local_t, inside = ctx.saved_tensors
        rows = e.shape[0]
        g = e / s[:, None]
        idx = torch.nonzero(inside, as_tuple=True)[0]
        g[idx, local_t[idx]] -= 1.0
        g.mul_(d_loss / rows)
        out = torch.zeros(ctx.shape, dtype=ctx.dtype, device=e.device)
        out[:, : ctx.vocab_local] = g.to(ctx.dtype)
        return out, None, None, None, None


def _rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


class TPBlock(nn.Module):
    def __init__(self, spec: DecoderSpec, layer: int, tp: TensorParallel):
        super().__init__()
        self.spec, self.layer, self.tp = spec, layer, tp
        R = tp.world
        if spec.heads % R or spec.kv_heads % R or spec.ff_dim % R:
            raise ValueError(f"heads ({spec.heads}), kv heads ({spec.kv_heads}) and ff_dim ({spec.ff_dim}) must divide "
                             f"by the tensor-parallel size {R}")
        if spec.qk_norm or spec.post_norms or spec.parallel_blocks or spec.is_expert_layer(layer) or \
                spec.is_windowed(layer) or spec.attention_softcap is not None:
            raise NotImplementedError("tensor parallelism covers plain pre-norm blocks (no qk-norm, post-norms, "
                                      "parallel blocks, experts, windows or soft-capping)")
        self.Hl, self.Hkvl, self.D = spec.heads // R, spec.kv_heads // R, spec.head_dim
        self.ffl = spec.ff_dim // R
        dim = spec.dim
        mult = 2 if spec.gated else 1
        self.attn_norm = Norm(dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.mlp_norm = Norm(dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.qkv_weight = nn.Parameter(torch.empty((self.Hl + 2 * self.Hkvl) * self.D, dim))
        self.qkv_bias = nn.Parameter(torch.zeros((self.Hl + 2 * self.Hkvl) * self.D)) if spec.qkv_bias else None
        self.o_weight = nn.Parameter(torch.empty(dim, self.Hl * self.D))
        self.o_bias = nn.Parameter(torch.zeros(dim)) if spec.output_bias else None
        self.up_weight = nn.Parameter(torch.empty(mult * self.ffl, dim))
        self.up_bias = nn.Parameter(torch.zeros(mult * self.ffl)) if spec.feed_forward_bias else None
        self.down_weight = nn.Parameter(torch.empty(dim, self.ffl))
        self.down_bias = nn.Parameter(torch.zeros(dim)) if spec.feed_forward_bias else None
        self.scale = spec.attention_scale if spec.attention_scale is not None else 1.0 / math.sqrt(self.D)

    def replicated(self) -> List[nn.Parameter]:
        ps = list(self.attn_norm.parameters()) + list(self.mlp_norm.parameters())
        return ps + [p for p in (self.o_bias, self.down_bias) if p is not None]

    @torch.no_grad()
    def load_from(self, blk) -> None:
        s, r, R = self.spec, self.tp.rank, self.tp.world
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim

        def qkv_rows(t):
            q, k, v = t[: H * D], t[H * D: (H + Hkv) * D], t[(H + Hkv) * D:]
            return torch.cat([_rows(q, r, R), _rows(k, r, R), _rows(v, r, R)], 0)

        a, m = blk.attn, blk.mlp
        self.qkv_weight.copy_(qkv_rows(a.qkv_weight))
        if self.qkv_bias is not None:
            self.qkv_bias.copy_(qkv_rows(a.qkv_bias))
        self.o_weight.copy_(_rows(a.o_weight.t(), r, R).t())
        if self.o_bias is not None:
            self.o_bias.copy_(a.o_bias)
        ff = s.ff_dim
        if s.gated:
            self.up_weight.copy_(torch.cat([_rows(m.up_weight[:ff], r, R), _rows(m.up_weight[ff:], r, R)], 0))
            if self.up_bias is not None:
                self.up_bias.copy_(torch.cat([_rows(m.up_bias[:ff], r, R), _rows(m.up_bias[ff:], r, R)], 0))
        else:
            self.up_weight.copy_(_rows(m.up_weight, r, R))
            if self.up_bias is not None:
                self.up_bias.copy_(_rows(m.up_bias, r, R))
        self.down_weight.copy_(_rows(m.down_weight.t(), r, R).t())
        if self.down_bias is not None:
            self.down_bias.copy_(m.down_bias)
        self.attn_norm.load_state_dict(blk.attn_norm.state_dict())
        self.mlp_norm.load_state_dict(blk.mlp_norm.state_dict())

    def forward(self, x_local, B: int, S: int, positions=None):
        s, tp = self.spec, self.tp
        h = self.attn_norm(x_local)
        qkv = column_parallel_linear(h, self.qkv_weight, self.qkv_bias, tp)
        rope = s.rope
        if rope is not None and rope.scaling is not None:
            raise NotImplementedError("scaled RoPE tables under tensor parallelism")
        theta = rope.theta if rope is not None else None
        rdim = rope.rotary_dim if rope is not None else None
        a = ops.qkv_attention(qkv.view(B, S, -1), self.Hl, self.Hkvl, self.D, True, self.scale, theta, rdim, 1.0,
                              positions)
        x_local = row_parallel_linear(a.reshape(B * S, -1), self.o_weight, self.o_bias, x_local, tp)
        h = self.mlp_norm(x_local)
        u = column_parallel_linear(h, self.up_weight, self.up_bias, tp)
        if s.gated:
            kind = {"silu": "silu", "gelu": "gelu", "relu": "relu"}.get(s.activation)
            if kind is None:
                raise NotImplementedError(f"gated activation '{s.activation}' under tensor parallelism")
            mid = ops.gated_activation(u, kind)
        else:
            mid = ops.gelu(u) if s.activation == "gelu" else (torch.relu(u) if s.activation == "relu"
                                                              else torch.nn.functional.silu(u))
        return row_parallel_linear(mid, self.down_weight, self.down_bias, x_local, tp)


class TPDecoder(nn.Module):
    """The decoder of ``spec`` sliced for one tensor-parallel rank."""

    def __init__(self, spec: DecoderSpec, tp: TensorParallel):
        super().__init__()
        self.spec, self.tp = spec, tp
        R = tp.world
        vp = spec.padded_vocabulary
        if vp % (R * 8):
            raise ValueError(f"the padded vocabulary ({vp}) must divide by 8 x the tensor-parallel size ({R})")
        self.vocab_rows = vp // R
        self.first = tp.rank * self.vocab_rows
        self.vocab_local = max(0, min(self.vocab_rows, spec.vocabulary - self.first))
        self.embed = nn.Parameter(torch.empty(self.vocab_rows, spec.dim))
        self.pos = nn.Parameter(torch.empty(spec.max_positions, spec.dim)) if spec.learned_positions else None
        self.blocks = nn.ModuleList([TPBlock(spec, i, tp) for i in range(spec.layers)])
        self.norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.head = None if spec.tie_embeddings else nn.Parameter(torch.empty(self.vocab_rows, spec.dim))
        if spec.head_bias or spec.logit_softcap:
            raise NotImplementedError("head bias / logit soft-capping under tensor parallelism")

    @classmethod
    def from_decoder(cls, model: Decoder, tp: TensorParallel) -> "TPDecoder":
        """Slice ``model`` (the same full model on every rank, e.g. freshly loaded) for this rank."""
        p = next(model.parameters())
        out = cls(model.spec, tp).to(p.device, p.dtype)
        with torch.no_grad():
            out.embed.copy_(_rows(model.embed, tp.rank, tp.world))
            if out.pos is not None:
                out.pos.copy_(model.pos)
            if out.head is not None:
                out.head.copy_(_rows(model.head, tp.rank, tp.world))
            out.norm.load_state_dict(model.norm.state_dict())
            for mine, blk in zip(out.blocks, model.blocks):
                mine.load_from(blk)
        return out

    def replicated(self) -> List[nn.Parameter]:
        ps = list(self.norm.parameters()) + ([self.pos] if self.pos is not None else [])
        for b in self.blocks:
            ps += b.replicated()
        return ps

    def sharded(self) -> List[nn.Parameter]:
        rep = {id(p) for p in self.replicated()}
        return [p for p in self.parameters() if id(p) not in rep]

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of replicated parameters over the ranks (each rank saw only its rows)."""
        if self.tp.world == 1:
            return
        grads = [p.grad for p in self.replicated() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=self.tp.group)
        off = 0
        for g in grads:
            g.copy_(flat[off: off + g.numel()].view_as(g))
            off += g.numel()

    def hidden_local(self, ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        spec, tp = self.spec, self.tp
        B, S = ids.shape
        M = B * S
        if M % tp.world:
            raise ValueError(f"batch x sequence ({M}) must divide by the tensor-parallel size ({tp.world})")
        x = _VocabParallelEmbedding.apply(ids.reshape(-1), self.embed, self.first, tp)
        if self.pos is not None:
            pos = positions.reshape(-1).long() if positions is not None else \
                torch.arange(S, device=ids.device).repeat(B)
            x = x + self.pos[_rows(pos, tp.rank, tp.world)]
        if spec.embedding_scale is not None:
            x = x * spec.embedding_scale
        for blk in self.blocks:
            x = blk(x, B, S, positions)
        return self.norm(x)

    def loss(self, ids: torch.Tensor, targets: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = self.hidden_local(ids, positions)
        w = self.embed if self.head is None else self.head
        logits = column_parallel_linear(h, w, None, self.tp)
        return _VocabParallelCrossEntropy.apply(logits, targets.reshape(-1), self.first, self.vocab_local, self.tp.group)

    def decay_groups(self, weight_decay: float):
        decay = [p for p in self.parameters() if p.dim() >= 2]
        rest = [p for p in self.parameters() if p.dim() < 2]
        return [{"params": decay, "weight_decay": weight_decay}, {"params": rest, "weight_decay": 0.0}]


class TPOptimizer:
    """AdamW over this rank's slice with the clip factor taken from the global gradient norm: sharded parameters
    count once per rank, replicated ones once in total."""

    def __init__(self, model: TPDecoder, lr: float = 3e-4, weight_decay: float = 0.1, max_grad_norm: float = 1.0, **kw):
        self.model = model
        self.inner = ops.FusedAdamW(model.decay_groups(weight_decay), lr=lr, weight_decay=weight_decay,
                                    max_grad_norm=max_grad_norm, **kw)

    def zero_grad(self):
        self.inner.zero_grad()

    @torch.no_grad()
    def step(self):
        m, tp = self.model, self.model.tp
        m.sync_replicated_grads()
        extra = None
        if tp.world > 1:
            sq = lambda ps: sum((p.grad.float().pow(2).sum() for p in ps if p.grad is not None),
                                torch.zeros((), device=m.embed.device))
            sharded, rep = sq(m.sharded()), sq(m.replicated())
            total = sharded + rep / tp.world
            dist.all_reduce(total, group=tp.group)
            extra = (total - sharded - rep).reshape(1).float()      # what the other ranks add to this rank's own sum
        self.inner.step(extra_sumsq=extra)
