"""Runs a decoder over the paged KV cache: packed prefill of several prompts, and batched one-token decode.

Prefill packs the uncached tokens of every admitted prompt into one ``[1, T, dim]`` activation so each
projection is a single GEMM; attention then runs per prompt (flash kernel over that prompt's keys) and the
keys / values go to the prompt's cache blocks. Decode advances every running sequence by one token: one
GEMM per projection over ``[n, dim]``, in-place RoPE at each sequence's position, a paged cache write, the
split-KV decode-attention kernel over the block tables, the head GEMM, and the device sampler - the host
reads one int per sequence and nothing else.

Model features outside the kernels' fast path (attention soft-capping, scaled RoPE tables, query/key norms)
are composed from primitives around the same cache; numerics equal the training forward.

Reference: TextGenerator's prefill / decode loop (src/Idrak/Generation/TextGenerator.cs:569-623), KeyValueCache and
decode primitives (src/Idrak.Abstraction/Generation/Decoding.cs:243, Tensors/Tensor.Decoding.cs).
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..models.decoder import Decoder, FeedForward, apply_rope_table, masked_attention, project
from ..ops import decode as dops


@dataclass
class PrefillItem:
    tokens: List[int]          # the tokens to compute (positions start .. start + len - 1)
    start: int                 # number of leading tokens already in the cache (shared prefix)
    blocks: List[int]          # block table covering positions 0 .. start + len


def fold_norms_into_projections(model: Decoder) -> bool:
    """Rewrites an inference copy of a pre-norm decoder so that every RMS norm's weight lives in the projection that
    follows it (query/key/value, gate/up, the head) and the norm itself has unit weight: ``norm(x) W^T`` becomes
    ``(x rstd) (W diag(w))^T``. Same function up to bf16 rounding of the folded weights, for every path (prefill, decode,
    training forward), and it lets the few-row decode kernel apply ``rstd`` in its epilogue instead of a norm launch.
    Returns False (and changes nothing) for models it does not cover: LayerNorm, post-norms, parallel blocks, experts,
    adapters or packed weights, tied embeddings (the head shares the embedding matrix)."""
    s = model.spec
    if getattr(model, "_norms_folded", False):
        return True
    if s.norm != "rms" or s.post_norms or s.parallel_blocks or s.experts > 0 or model.head is None:
        return False
    from ..ops.skinny import fold_norm
    blocks = list(model.blocks)
    for blk in blocks:
        if any(getattr(m, "adapters", None) is not None or getattr(m, "packed", None) for m in (blk.attn, blk.mlp)):
            return False
    with torch.no_grad():
        def fold(weight: torch.nn.Parameter, norm) -> None:
            weight.copy_(fold_norm(weight, norm.effective_weight()))
            norm.weight.fill_(1.0 - (s.norm_offset or 0.0))          # effective weight 1 from here on
        for blk in blocks:
            fold(blk.attn.qkv_weight, blk.attn_norm)
            fold(blk.mlp.up_weight, blk.mlp_norm)
        fold(model.head, model.norm)
    model._norms_folded = True
    return True


class ModelRunner:
    def __init__(self, model: Decoder, num_blocks: int, block_size: int = 16, max_batch: int = 256,
                 cache_dtype: Optional[torch.dtype] = None):
        self.model = model.eval()
        self.spec = model.spec
        p = next(model.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.block_size, self.num_blocks, self.max_batch = block_size, num_blocks, max_batch
        s = self.spec
        cd = cache_dtype or self.dtype
        # one block more than the scheduler hands out: padding rows of a graph-replayed decode batch write there
        self.k_cache = [torch.zeros(num_blocks + 1, block_size, s.kv_heads, s.head_dim, dtype=cd, device=self.device)
                        for _ in range(s.layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        # an int8 cache keeps one fp32 scale per (slot, kv head) beside the codes
        self.kv_int8 = cd == torch.int8
        self.k_scale = self.v_scale = [None] * s.layers
        if self.kv_int8:
            self.k_scale = [torch.zeros(num_blocks + 1, block_size, s.kv_heads, dtype=torch.float32, device=self.device)
                            for _ in range(s.layers)]
            self.v_scale = [torch.zeros_like(k) for k in self.k_scale]
        self.trash_block = num_blocks
        self.max_blocks_per_seq = (s.max_positions + block_size - 1) // block_size
        self._graphs = {}
        self._graph_pool = None
        self.graph_replays = 0

    # ------------------------------------------------------------------ sizing
    @staticmethod
    def blocks_that_fit(spec, bytes_available: int, block_size: int = 16, elem_bytes: int = 2) -> int:
        per_block = 2 * spec.layers * block_size * spec.kv_heads * (spec.head_dim * elem_bytes + (4 if elem_bytes == 1 else 0))
        return max(int(bytes_available // per_block), 1)

    # ------------------------------------------------------------------ shared pieces
    def _embed(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        m, s = self.model, self.spec
        x = ops.embedding(ids.view(1, -1), m.embed, None)
        if m.pos is not None:
            x = x + m.pos[positions.long()][None]
        if s.embedding_scale is not None:
            x = x * s.embedding_scale
        return x

    def _qkv(self, attn, x):
        adapters = getattr(attn, "adapters", None)
        packed = getattr(attn, "packed", {})
        if adapters is not None:
            from ..adapters.lora import _slices_attention, project_with_adapters
            qkv = project_with_adapters(x, attn.qkv_weight, attn.qkv_bias, adapters, _slices_attention(self.spec),
                                        packed=packed.get("qkv"))
            return qkv.contiguous()
        return project(x, attn.qkv_weight, packed.get("qkv"), attn.qkv_bias)

    def _out(self, attn, a, residual):
        adapters = getattr(attn, "adapters", None)
        packed = getattr(attn, "packed", {})
        if adapters is not None and "o" in adapters:
            from ..adapters.lora import project_with_adapters
            return project_with_adapters(a, attn.o_weight, attn.o_bias, adapters, {"o": (0, self.spec.dim)}, residual,
                                         packed=packed.get("o"))
        return project(a, attn.o_weight, packed.get("o"), attn.o_bias, residual)

    def _rotate_and_cache(self, attn, qkv2, positions, slots, li: int) -> None:
        """Query / key norms, RoPE (both in place on the packed projection) and the cache write of the new keys and
        values: one fused launch where the kernel covers the model's settings, the separate steps otherwise."""
        s = self.spec
        rope = attn.rope
        if rope is None or rope.scaling is None:
            qn = attn.q_norm.effective_weight() if s.qk_norm else None
            kn = attn.k_norm.effective_weight() if s.qk_norm else None
            dops.norm_rope_kv(qkv2, s.heads, s.kv_heads, s.head_dim, positions, slots, self.k_cache[li], self.v_cache[li],
                              self.k_scale[li], self.v_scale[li], qn, kn, s.norm_epsilon,
                              rope.theta if rope is not None else None, rope.rotary_dim if rope is not None else None)
            return
        self._rotate(attn, qkv2, positions)
        dops.norm_rope_kv(qkv2, s.heads, s.kv_heads, s.head_dim, None, slots, self.k_cache[li], self.v_cache[li],
                          self.k_scale[li], self.v_scale[li])

    def _cached_kv(self, li: int, blocks: torch.Tensor, total: int, dtype):
        """Keys and values of positions ``0 .. total`` of one sequence read back from its blocks: ``[1, total, Hkv, D]``."""
        s = self.spec
        k = self.k_cache[li][blocks].reshape(-1, s.kv_heads, s.head_dim)[:total]
        v = self.v_cache[li][blocks].reshape(-1, s.kv_heads, s.head_dim)[:total]
        if self.kv_int8:
            k = k.float() * self.k_scale[li][blocks].reshape(-1, s.kv_heads)[:total, :, None]
            v = v.float() * self.v_scale[li][blocks].reshape(-1, s.kv_heads)[:total, :, None]
        return k[None].to(dtype), v[None].to(dtype)

    def _rotate(self, attn, qkv2, positions):
        """RoPE (and query / key norms) in place on the packed ``[T, (H + 2 Hkv) D]`` projection."""
        s = self.spec
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim
        T = qkv2.shape[0]
        qk = qkv2[:, : (H + Hkv) * D].unflatten(-1, (H + Hkv, D))
        if s.qk_norm:
            q = attn.q_norm(qk[:, :H].contiguous())
            k = attn.k_norm(qk[:, H:].contiguous())
            qk[:, :H].copy_(q)
            qk[:, H:].copy_(k)
        rope = attn.rope
        if rope is None:
            return
        if rope.scaling is None:
            ops.rope_(qk, positions, rope.theta, rope.rotary_dim, 1.0)
        else:
            r = apply_rope_table(qk[None], rope, positions[None])
            qk.copy_(r[0])

    def _block(self, blk, x, attend):
        """One decoder block around ``attend(attn_module, normed_x, residual_or_None)``; mirrors DecoderBlock.forward."""
        s = self.spec
        if s.parallel_blocks:
            h = blk.attn_norm(x)
            return x + attend(blk.attn, h, None) + blk.mlp(h)
        if s.post_norms:
            a = blk.post_attn_norm(attend(blk.attn, blk.attn_norm(x), None))
            x = x + a
            return x + blk.post_mlp_norm(blk.mlp(blk.mlp_norm(x)))
        x = attend(blk.attn, blk.attn_norm(x), x)
        return blk.mlp(blk.mlp_norm(x), x)

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        """``[rows, padded vocabulary]`` logits of already-normalised hidden rows."""
        m, s = self.model, self.spec
        logits = ops.linear(h, m.head_weight(), m.head_bias)
        if s.logit_softcap:
            c = s.logit_softcap
            logits = torch.tanh(logits.float() / c).mul(c).to(logits.dtype)
        return logits.reshape(-1, logits.shape[-1])

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, items: Sequence[PrefillItem], all_logits: bool = False) -> torch.Tensor:
        """Computes the listed tokens of every item, fills the cache, and returns the logits of each item's last
        token ``[len(items), padded vocabulary]`` (or of every computed token, packed, when ``all_logits``)."""
        s, dev, bs = self.spec, self.device, self.block_size
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim
        ids, pos, slots, bounds = [], [], [], [0]
        for it in items:
            n = len(it.tokens)
            ids += it.tokens
            for j in range(n):
                p = it.start + j
                pos.append(p)
                slots.append(it.blocks[p // bs] * bs + p % bs)
            bounds.append(bounds[-1] + n)
        ids_t = torch.tensor(ids, dtype=torch.int32, device=dev)
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slots_t = torch.tensor(slots, dtype=torch.int32, device=dev)
        tables = [torch.tensor(it.blocks, dtype=torch.long, device=dev) if it.start > 0 else None for it in items]
        x = self._embed(ids_t, pos_t)
        layer_index = {id(blk.attn): i for i, blk in enumerate(self.model.blocks)}
        runs = []                                  # (first item, count, length) of >= 2 fresh prompts of equal length
        i = 0
        while i < len(items):
            j = i
            while (j + 1 < len(items) and items[j + 1].start == 0 and items[i].start == 0
                   and len(items[j + 1].tokens) == len(items[i].tokens)):
                j += 1
            if j > i and len(items[i].tokens) % 8 == 0:
                runs.append((i, j - i + 1, len(items[i].tokens)))
            i = j + 1

        def attend(attn, h, residual):
            li = layer_index[id(attn)]
            qkv = self._qkv(attn, h)
            qkv2 = qkv.view(-1, qkv.shape[-1])
            self._rotate_and_cache(attn, qkv2, pos_t, slots_t, li)
            q = qkv2[:, : H * D].unflatten(-1, (H, D))
            k = qkv2[:, H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
            v = qkv2[:, (H + Hkv) * D:].unflatten(-1, (Hkv, D))
            window = s.sliding_window if s.is_windowed(attn.layer) else None
            fast = window is None and s.attention_softcap is None
            out = torch.empty(qkv2.shape[0], H * D, dtype=qkv.dtype, device=dev)
            done = set()
            if fast:
                # runs of fresh prompts of one length are contiguous in the pack: one batched attention launch
                for first, count, length in runs:
                    a, b = bounds[first], bounds[first + count]
                    o = ops.attention(q[a:b].unflatten(0, (count, length)), k[a:b].unflatten(0, (count, length)),
                                      v[a:b].unflatten(0, (count, length)), True, attn.scale)
                    out[a:b] = o.reshape(b - a, H * D)
                    done.update(range(first, first + count))
            for i, it in enumerate(items):
                if i in done:
                    continue
                a, b = bounds[i], bounds[i + 1]
                qi = q[a:b][None]
                if it.start > 0:     # queries see the shared prefix too: read keys / values back from the cache
                    total = it.start + (b - a)
                    ki, vi = self._cached_kv(li, tables[i], total, qkv.dtype)
                else:
                    ki, vi = k[a:b][None], v[a:b][None]
                if fast:
                    o = ops.attention(qi, ki, vi, True, attn.scale)
                else:
                    o = masked_attention(qi, ki, vi, attn.scale, window, s.attention_softcap)
                out[a:b] = o.reshape(b - a, H * D)
            return self._out(attn, out[None], residual)

        for blk in self.model.blocks:
            x = self._block(blk, x, attend)
        if all_logits:
            return self._logits(self.model.norm(x))
        last = torch.tensor([b - 1 for b in bounds[1:]], dtype=torch.long, device=dev)
        h = self.model.norm(x[0, last].contiguous()[None])
        return self._logits(h)

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def decode(self, tokens: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
               max_len_hint: Optional[int] = None) -> torch.Tensor:
        """One new token per sequence. ``tokens`` / ``positions`` int32 ``[n]`` (position = index of the new
        token), ``block_table`` int32 ``[n, max_blocks]``. Returns logits ``[n, padded vocabulary]``."""
        s, dev, bs = self.spec, self.device, self.block_size
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim
        n = tokens.shape[0]
        rows = torch.arange(n, device=dev)
        blk_of = block_table[rows, (positions // bs).long()]
        slots = (blk_of * bs + positions % bs).to(torch.int32)
        lens = (positions + 1).to(torch.int32)
        x = self._embed(tokens, positions)
        if n <= 64 and self._few_row_path():
            return self._decode_few_rows(x.view(n, -1), positions, slots, block_table, lens, max_len_hint)
        layer_index = {id(blk.attn): i for i, blk in enumerate(self.model.blocks)}

        def attend(attn, h, residual):
            li = layer_index[id(attn)]
            qkv = self._qkv(attn, h)
            qkv2 = qkv.view(-1, qkv.shape[-1])
            self._rotate_and_cache(attn, qkv2, positions, slots, li)
            q = qkv2[:, : H * D].unflatten(-1, (H, D))
            window = s.sliding_window if s.is_windowed(attn.layer) else 0
            if s.attention_softcap is None:
                o = dops.paged_decode(q, self.k_cache[li], self.v_cache[li], block_table, lens,
                                      attn.scale, window or 0, max_len_hint=max_len_hint,
                                      k_scale=self.k_scale[li], v_scale=self.v_scale[li])
            else:
                o = self._decode_softcap(q, li, block_table, lens, attn.scale, window or None)
            return self._out(attn, o.reshape(1, n, H * D), residual)

        for blk in self.model.blocks:
            x = self._block(blk, x, attend)
        return self._logits(self.model.norm(x))

    # ------------------------------------------------------------------ decode of at most 64 rows: fused projections
    def _few_row_path(self) -> bool:
        """Whether decode steps of up to 64 sequences run on the few-row kernels: one launch per projection with bias,
        residual add, gated activation and (with folded norms) the RMS norm inside it."""
        cached = getattr(self, "_few_rows_ok", None)
        if cached is not None:
            return cached
        from ..ops import skinny
        from .. import _native
        s = self.spec
        ok = (self.device.type == "cuda" and self.dtype == torch.bfloat16 and _native.has("idrak_skinny_gemm")
              and os.environ.get("IDRAK_FEW_ROW_DECODE", "1") != "0"
              and not s.parallel_blocks and not s.post_norms and s.experts == 0 and s.attention_softcap is None
              and s.gated and s.activation in skinny._KINDS and s.dim % 8 == 0 and s.ff_dim % 8 == 0
              and not s.logit_softcap)
        for blk in self.model.blocks:
            if not ok:
                break
            rope = blk.attn.rope
            ok = (not any(getattr(m, "adapters", None) is not None or getattr(m, "packed", None)
                          for m in (blk.attn, blk.mlp)) and (rope is None or rope.scaling is None))
        self._few_rows_ok = bool(ok)
        return self._few_rows_ok

    def _decode_few_rows(self, x, positions, slots, block_table, lens, max_len_hint):
        """Six or seven launches per layer: qkv (+norm) | norms of q, k + RoPE + cache write | paged attention
        (+ its merge) | out + residual | gate/up (+norm) + activation | down + residual."""
        from ..ops.skinny import few_row_linear, skinny_linear
        s, m = self.spec, self.model
        H, Hkv, D = s.heads, s.kv_heads, s.head_dim
        folded = bool(getattr(m, "_norms_folded", False))
        eps = s.norm_epsilon if folded else None
        n = x.shape[0]
        for li, blk in enumerate(m.blocks):
            attn, mlp = blk.attn, blk.mlp
            h = x if folded else blk.attn_norm(x)
            qkv = skinny_linear(h, attn.qkv_weight, attn.qkv_bias, norm_eps=eps)
            self._rotate_and_cache(attn, qkv, positions, slots, li)
            q = qkv[:, : H * D].unflatten(-1, (H, D))
            window = s.sliding_window if s.is_windowed(attn.layer) else 0
            o = dops.paged_decode(q, self.k_cache[li], self.v_cache[li], block_table, lens, attn.scale, window or 0,
                                  max_len_hint=max_len_hint, k_scale=self.k_scale[li], v_scale=self.v_scale[li])
            x = skinny_linear(o.reshape(n, H * D), attn.o_weight, attn.o_bias, residual=x)
            if folded:
                g = skinny_linear(x, mlp.up_weight, mlp.up_bias, gate=s.activation, norm_eps=eps)
            else:
                # the stacked gate / up matrix is wide enough for the dense kernel to stream it faster (measured:
                # 56 + 8 us against 74 us at 64 rows of the 8 B shape); the few-row kernel earns its place where the
                # norm is folded in as well
                gu = ops.gemm(blk.mlp_norm(x), mlp.up_weight, bias=mlp.up_bias)
                g = ops.gated_activation(gu, s.activation)
            x = skinny_linear(g, mlp.down_weight, mlp.down_bias, residual=x)
        if folded:
            logits = skinny_linear(x, m.head_weight(), m.head_bias, norm_eps=s.norm_epsilon)
        else:
            logits = few_row_linear(m.norm(x), m.head_weight(), m.head_bias)      # a wide head streams faster densely
        return logits.reshape(-1, logits.shape[-1])

    # ------------------------------------------------------------------ decode as a replayed CUDA graph
    BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    @torch.no_grad()
    def decode_graphed(self, tokens: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                       longest: int) -> torch.Tensor:
        """``decode`` recorded once per (batch bucket, context bucket) as a CUDA graph and replayed: a decode step is
        hundreds of small launches, and replaying them removes the host's share of the step. The batch is padded to
        the bucket with rows that write to a spare cache block; the context bucket fixes the key split of the
        attention kernel. Returns logits ``[n, padded vocabulary]`` (a view of the graph's output buffer)."""
        n = tokens.shape[0]
        bucket = next((b for b in self.BATCH_BUCKETS if b >= n), None)
        if bucket is None or self.device.type != "cuda" or self.spec.attention_softcap is not None:
            return self.decode(tokens, positions, block_table, max_len_hint=longest)
        ctx = 256
        while ctx < longest:
            ctx *= 2
        width = self.max_blocks_per_seq
        key = (bucket, ctx)
        entry = self._graphs.get(key)
        if entry is None:
            tok = torch.zeros(bucket, dtype=torch.int32, device=self.device)
            pos = torch.zeros(bucket, dtype=torch.int32, device=self.device)
            tab = torch.full((bucket, width), self.trash_block, dtype=torch.int32, device=self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                   # warm-up: lazy buffers and kernel attributes get created
                for _ in range(2):
                    self.decode(tok, pos, tab, max_len_hint=ctx)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                out = self.decode(tok, pos, tab, max_len_hint=ctx)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = self._graphs[key] = (graph, tok, pos, tab, out)
        graph, tok, pos, tab, out = entry
        tok[:n].copy_(tokens, non_blocking=True)
        pos[:n].copy_(positions, non_blocking=True)
        if n < bucket:
            tok[n:].zero_()
            pos[n:].zero_()
            tab[n:].fill_(self.trash_block)
        w = block_table.shape[1]
        tab[:n, :w].copy_(block_table, non_blocking=True)
        graph.replay()
        self.graph_replays += 1
        return out[:n]

    def _decode_softcap(self, q, li, block_table, lens, scale, window):
        """Soft-capped scores (Gemma-2 style) composed from primitives, one sequence at a time."""
        s = self.spec
        out = torch.empty_like(q)
        for i in range(q.shape[0]):
            n = int(lens[i])
            blocks = block_table[i, : (n + self.block_size - 1) // self.block_size].long()
            k, v = self._cached_kv(li, blocks, n, q.dtype)
            out[i] = masked_attention(q[i][None, None], k, v, scale, window, s.attention_softcap)[0, 0]
        return out

    # ------------------------------------------------------------------ embeddings endpoint
    @torch.no_grad()
    def embed_text(self, tokens: Sequence[int], pooling: str = "mean") -> torch.Tensor:
        """A sentence vector from the final hidden states (mean over tokens, or the last token), L2-normalised."""
        ids = torch.tensor([list(tokens)], dtype=torch.int32, device=self.device)
        h = self.model.hidden(ids).float()[0]
        v = h.mean(0) if pooling == "mean" else h[-1]
        return torch.nn.functional.normalize(v, dim=0)
