"""``ModelRunner`` over a tensor-parallel slice of the decoder.

Every rank of the group runs this runner in lock-step over its own heads, feed-forward columns and paged KV cache
(``parallel.tp_serve.shard_decoder``). The attention output projection and the feed-forward down projection produce
partial rows; ``TPServeContext.all_reduce_rows`` sums them across the ranks inside one peer-memory kernel that also
adds the residual and applies the following norm. Prefill steps with many rows use the two-shot all-reduce (reduce-
scatter then all-gather, 2 (W-1)/W of the bytes per rank instead of W-1 times them). The head yields this rank's
slice of the vocabulary; ``LLMEngine`` merges arg-maxima or gathers the slices before sampling.

Reference: the single-device decode step it splits is TextGenerator's (src/Idrak/Generation/TextGenerator.cs:1148-1201).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..parallel.tp_serve import TPServeContext, vocab_slice
from .runner import ModelRunner

ONE_SHOT_ROWS = 256          # above this many rows the two-shot all-reduce moves fewer bytes per rank


class TPModelRunner(ModelRunner):
    def __init__(self, model, num_blocks: int, block_size: int = 16, max_batch: int = 256,
                 cache_dtype: Optional[torch.dtype] = None, tp: Optional[TPServeContext] = None):
        if tp is None:
            raise ValueError("TPModelRunner needs the group's TPServeContext")
        if not hasattr(model, "tp_head"):
            raise ValueError("the model is not a tensor-parallel slice (see parallel.tp_serve.shard_decoder)")
        super().__init__(model, num_blocks, block_size, max_batch, cache_dtype)
        self.tp = tp
        self.full_spec = model.tp_full_spec
        lo, hi = vocab_slice(self.full_spec, tp.rank, tp.world)
        self.vocab_offset = lo
        self.vocab_local = max(0, min(hi, self.full_spec.vocabulary) - lo)      # columns of the slice that are real tokens

    def _few_row_path(self) -> bool:
        """Decode steps of up to 64 sequences on the few-row projection kernels, as on one GPU, with the row-parallel
        products written straight into the symmetric buffer the all-reduce kernel reads."""
        import os
        return os.environ.get("IDRAK_TP_FEW_ROW_DECODE", "1") != "0" and super()._few_row_path()

    def _decode_few_rows(self, x, positions, slots, block_table, lens, max_len_hint):
        """Eight or nine launches per layer: qkv | q/k norms + RoPE + cache write | paged attention (+ merge) | out
        (partial, into the symmetric buffer) | all-reduce + residual + norm | gate/up + activation | down (partial) |
        all-reduce + residual + the next layer's norm."""
        from ..ops import decode as dops
        from ..ops.skinny import few_row_linear, skinny_linear
        s, m, tp = self.spec, self.model, self.tp
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim
        n = x.shape[0]
        blocks = list(m.blocks)
        h = blocks[0].attn_norm(x)
        for li, blk in enumerate(blocks):
            attn, mlp = blk.attn, blk.mlp
            qkv = skinny_linear(h, attn.qkv_weight, attn.qkv_bias)
            self._rotate_and_cache(attn, qkv, positions, slots, li)
            q = qkv[:, : H * D].unflatten(-1, (H, D))
            window = s.sliding_window if s.is_windowed(attn.layer) else 0
            o = dops.paged_decode(q, self.k_cache[li], self.v_cache[li], block_table, lens, attn.scale, window or 0,
                                  max_len_hint=max_len_hint, k_scale=self.k_scale[li], v_scale=self.v_scale[li])
            part = skinny_linear(o.reshape(n, H * D), attn.o_weight, attn.o_bias, out=tp.partial_buffer(n))
            x, h = tp.all_reduce_rows(part, x, blk.mlp_norm)
            g = few_row_linear(h, mlp.up_weight, mlp.up_bias, gate=s.activation)
            part = skinny_linear(g, mlp.down_weight, mlp.down_bias, out=tp.partial_buffer(n))
            nxt = blocks[li + 1].attn_norm if li + 1 < len(blocks) else m.norm
            x, h = tp.all_reduce_rows(part, x, nxt)
        logits = few_row_linear(h, m.tp_head, m.tp_head_bias)
        return logits.reshape(-1, logits.shape[-1])

    def _sum_partials(self, partial: torch.Tensor, residual: torch.Tensor, norm=None):
        """``residual + sum over ranks(partial)`` (and the norm of that): ``[1, T, dim]`` in and out."""
        shape = partial.shape
        dim = shape[-1]
        p2, r2 = partial.reshape(-1, dim), residual.reshape(-1, dim)
        rows = p2.shape[0]
        if rows <= ONE_SHOT_ROWS:
            x, h = self.tp.all_reduce_rows(p2, r2, norm)
            return x.view(shape), (h.view(shape) if h is not None else None)
        # many rows (prefill): in-place two-shot all-reduce over the symmetric buffer, then the element-wise tail
        view = self.tp.partial_buffer(rows)
        view.copy_(p2)
        buf = self.tp._bufs[self.tp._turn]
        self.tp._turn ^= 1
        pad = (-rows * dim) % (self.tp.world * 8)
        self.tp.comm.all_reduce(buf, torch.bfloat16, rows * dim + pad)
        x = ops.add(view, r2).view(shape)
        return x, (norm(x) if norm is not None else None)

    def _block(self, blk, x, attend):
        a = attend(blk.attn, blk.attn_norm(x), None)                 # this rank's heads: a partial sum over ranks
        x, h = self._sum_partials(a, x, blk.mlp_norm)
        m = blk.mlp(h, None)                                          # this rank's feed-forward columns
        x, _ = self._sum_partials(m, x, None)
        return x

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        """This rank's vocabulary slice ``[rows, padded vocabulary / world]``."""
        m, s = self.model, self.spec
        logits = ops.linear(h, m.tp_head, m.tp_head_bias)
        if s.logit_softcap:
            c = s.logit_softcap
            logits = torch.tanh(logits.float() / c).mul(c).to(logits.dtype)
        return logits.reshape(-1, logits.shape[-1])
