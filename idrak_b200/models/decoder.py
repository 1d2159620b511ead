"""The decoder-only transformer every supported family is an instance of, built from a ``DecoderSpec``.

Parameters are kept in the layout the kernels want: one packed QKV projection ``[(H + 2*Hkv)*D, dim]``,
one packed gate/up projection ``[2*ff, dim]`` (``nn.Linear`` orientation, K-major for the GEMM), an
embedding table padded to a multiple of 64 rows. ``checkpoint_names`` maps these to the reference's
per-matrix names and ``[in, out]`` orientation for file I/O.

Training forward on the GPU goes through the fused functions of ``idrak_b200.ops`` (bias / GELU /
residual inside GEMM epilogues, RoPE in place, flash attention, chunked head + loss). The same module
runs on the CPU in fp32 with plain PyTorch math.

Reference: DecoderBuilder.Build (src/Idrak/Layers/DecoderBuilder.cs:23), CausalSelfAttention /
FeedForward / DecoderBlock (src/Idrak/Layers/Decoder.cs:108,820,969), PositionEmbedding (:1251).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .. import ops
from .spec import DecoderSpec


class Norm(nn.Module):
    def __init__(self, dim: int, kind: str, eps: float, offset: float = 0.0):
        super().__init__()
        self.kind, self.eps, self.offset = kind, eps, offset
        self.weight = nn.Parameter(torch.ones(dim) if offset == 0.0 else torch.zeros(dim))
        self.bias = nn.Parameter(torch.zeros(dim)) if kind == "layer" else None

    def effective_weight(self):
        return self.weight if self.offset == 0.0 else self.weight + self.offset

    def forward(self, x):
        w = self.effective_weight()
        if self.kind == "layer":
            return ops.layer_norm(x, w, self.bias, self.eps)
        return ops.rms_norm(x, w, self.eps)

    def branch(self, x):
        """``(norm(x), x)`` for a pre-norm residual block; see ``ops.norm_branch``."""
        return ops.norm_branch(x, self.effective_weight(), self.bias, self.eps, self.kind != "layer")


def project(x, weight, packed, bias=None, residual=None):
    """``x W^T + b (+ residual)`` over the dense weight, or over its packed int8 / int4 replacement."""
    if packed is not None:
        from ..quant.weights import qlinear
        return qlinear(x, packed, bias, residual)
    return ops.linear(x, weight, bias, residual)


class SelfAttention(nn.Module):
    def __init__(self, spec: DecoderSpec, layer: int):
        super().__init__()
        self.spec, self.layer = spec, layer
        H, Hkv, D, dim = spec.heads, spec.kv_heads, spec.head_dim, spec.dim
        self.qkv_weight = nn.Parameter(torch.empty((H + 2 * Hkv) * D, dim))
        self.qkv_bias = nn.Parameter(torch.zeros((H + 2 * Hkv) * D)) if spec.qkv_bias else None
        self.o_weight = nn.Parameter(torch.empty(dim, H * D))
        self.o_bias = nn.Parameter(torch.zeros(dim)) if spec.output_bias else None
        if spec.qk_norm:
            self.q_norm = Norm(D, "rms", spec.norm_epsilon, spec.norm_offset)
            self.k_norm = Norm(D, "rms", spec.norm_epsilon, spec.norm_offset)
        self.scale = spec.attention_scale if spec.attention_scale is not None else 1.0 / math.sqrt(D)
        rope = spec.sliding_window_rope if (spec.is_windowed(layer) and spec.sliding_window_rope) else spec.rope
        self.rope = rope

    def forward(self, x, residual=None, positions=None, spans=None):
        spec = self.spec
        H, Hkv, D = spec.heads, spec.kv_heads, spec.head_dim
        adapters = getattr(self, "adapters", None)
        packed = getattr(self, "packed", {})
        if adapters is not None:
            from ..adapters.lora import _slices_attention, project_with_adapters
            qkv = project_with_adapters(x, self.qkv_weight, self.qkv_bias, adapters, _slices_attention(spec),
                                        packed=packed.get("qkv"))
            if not qkv.is_contiguous():
                qkv = qkv.contiguous()
        else:
            qkv = project(x, self.qkv_weight, packed.get("qkv"), self.qkv_bias)
        window = spec.sliding_window if spec.is_windowed(self.layer) else None
        # sequences packed into one row: one launch, every position bounded below by the start of its own sequence
        row_start = None
        if spans is not None:
            row_start = spans if torch.is_tensor(spans) else ops.row_starts_from_spans(
                spans, qkv.shape[0], qkv.shape[1], qkv.device)
        simple = not spec.qk_norm and (self.rope is None or self.rope.scaling is None)
        if simple:
            theta = self.rope.theta if self.rope is not None else None
            rdim = self.rope.rotary_dim if self.rope is not None else None
            a = ops.qkv_attention(qkv, H, Hkv, D, True, self.scale, theta, rdim, 1.0, positions, window, row_start,
                                  spec.attention_softcap)
        else:
            a = self._general(qkv, positions, window, row_start)
        if adapters is not None and "o" in adapters:
            from ..adapters.lora import project_with_adapters
            return project_with_adapters(a, self.o_weight, self.o_bias, adapters,
                                         {"o": (0, spec.dim)}, residual, packed=packed.get("o"))
        return project(a, self.o_weight, packed.get("o"), self.o_bias, residual)

    def _general(self, qkv, positions, window, row_start=None):
        """qk-norm and scaled RoPE tables ahead of the attention kernel."""
        from ..ops.fused import _split_qkv
        spec = self.spec
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, spec.heads, spec.kv_heads, spec.head_dim)
        if spec.qk_norm:
            q, k = self.q_norm(q.contiguous()), self.k_norm(k.contiguous())
        if self.rope is not None:
            q, k = apply_rope_table(q, self.rope, positions), apply_rope_table(k, self.rope, positions)
        a = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), True, self.scale, window, row_start,
                          spec.attention_softcap)
        return a.reshape(B, S, spec.heads * spec.head_dim)


def apply_rope_table(x, rope, positions=None):
    """RoPE with an explicit (possibly scaled) frequency table; x: [B, S, H, D]. Differentiable."""
    B, S, H, D = x.shape
    inv, mscale = rope.inv_freq(D, S)
    rot = rope.rotary_dim or D
    half = rot // 2
    inv_t = torch.tensor(inv, device=x.device, dtype=torch.float32)
    pos = (positions.reshape(B, S).float() if positions is not None
           else torch.arange(S, device=x.device, dtype=torch.float32)[None, :].expand(B, S))
    ang = pos[..., None] * inv_t
    c, s = (torch.cos(ang) * mscale)[:, :, None, :], (torch.sin(ang) * mscale)[:, :, None, :]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = torch.cat([a * c - b * s, b * c + a * s, xf[..., rot:]], dim=-1)
    return out.to(x.dtype)


def masked_attention(q, k, v, scale, window=None, softcap=None):
    """Causal attention with a sliding window and/or tanh soft-capping (fp32 math): the oracle of the kernels' modes."""
    return ops.attention_reference(q, k, v, True, scale, window, None, softcap)


class FeedForward(nn.Module):
    def __init__(self, spec: DecoderSpec, ff_dim: Optional[int] = None):
        super().__init__()
        self.spec = spec
        ff = ff_dim or spec.ff_dim
        self.hidden = ff
        mult = 2 if spec.gated else 1
        self.up_weight = nn.Parameter(torch.empty(mult * ff, spec.dim))      # gated: [gate; up]
        self.up_bias = nn.Parameter(torch.zeros(mult * ff)) if spec.feed_forward_bias else None
        self.down_weight = nn.Parameter(torch.empty(spec.dim, ff))
        self.down_bias = nn.Parameter(torch.zeros(spec.dim)) if spec.feed_forward_bias else None

    def forward(self, x, residual=None):
        spec = self.spec
        adapters = getattr(self, "adapters", None)
        packed = getattr(self, "packed", {})
        if (adapters is not None and len(adapters.items) > 0) or packed:
            return self._forward_adapted(x, residual, adapters, packed)
        if spec.gated:
            kind = {"silu": "silu", "gelu": "gelu", "relu": "relu"}.get(spec.activation)
            if kind is None:   # tanh(gate) * sigmoid(up)
                gu = ops.linear(x, self.up_weight, self.up_bias)
                ff = gu.shape[-1] // 2
                h = torch.tanh(gu[..., :ff]) * torch.sigmoid(gu[..., ff:])
                return ops.linear(h, self.down_weight, self.down_bias, residual)
            return ops.mlp_gated(x, self.up_weight, self.up_bias, self.down_weight, self.down_bias, residual, kind)
        if spec.activation == "gelu":
            return ops.mlp_gelu(x, self.up_weight, self.up_bias, self.down_weight, self.down_bias, residual)
        h = ops.linear(x, self.up_weight, self.up_bias)
        h = torch.relu(h) if spec.activation == "relu" else torch.nn.functional.silu(h)
        return ops.linear(h, self.down_weight, self.down_bias, residual)


    def _forward_adapted(self, x, residual, adapters, packed=None):
        """The same block with low-rank adapters on gate / up / down and / or a packed (int8 / int4) base:
        projections run one by one."""
        from ..adapters.lora import project_with_adapters
        spec = self.spec
        packed = packed or {}
        hidden = self.hidden
        if spec.gated:
            gu = project_with_adapters(x, self.up_weight, self.up_bias, adapters,
                                       {"gate": (0, hidden), "up": (hidden, 2 * hidden)}, packed=packed.get("up"))
            kind = {"silu": "silu", "gelu": "gelu", "relu": "relu"}.get(spec.activation)
            if kind is None:
                h = torch.tanh(gu[..., :hidden]) * torch.sigmoid(gu[..., hidden:])
            else:
                h = ops.gated_activation(gu.contiguous(), kind)
        else:
            h = project_with_adapters(x, self.up_weight, self.up_bias, adapters, {"up": (0, hidden)},
                                      packed=packed.get("up"))
            h = ops.gelu(h) if spec.activation == "gelu" else (
                torch.relu(h) if spec.activation == "relu" else torch.nn.functional.silu(h))
        return project_with_adapters(h, self.down_weight, self.down_bias, adapters,
                                     {"down": (0, spec.dim)}, residual, packed=packed.get("down"))


class _AsStacked(torch.autograd.Function):
    """The stacked buffer as a function of the per-expert parameters that are views of its slices: forward hands out the
    buffer (no copy), backward splits the stacked gradient into one view per parameter."""

    @staticmethod
    def forward(ctx, buffer, *params):
        return buffer.view_as(buffer)

    @staticmethod
    def backward(ctx, grad):
        return (None,) + tuple(grad[i] for i in range(grad.shape[0]))


class MixtureOfExperts(nn.Module):
    """Top-k routed experts (+ optional shared expert). Single-device, as in the reference
    (src/Idrak/Layers/MixtureOfExperts.cs:34): ties go to the lowest index, weights optionally renormalised.

    The experts' matrices live side by side in two stacked buffers and every expert's parameter is a view of its slice,
    so checkpoints, optimizers and adapters keep seeing per-expert parameters while the device path (``ops.moe``:
    routing kernels + grouped tensor-core products, no host read) reads the stacked arrays."""

    def __init__(self, spec: DecoderSpec):
        super().__init__()
        self.spec = spec
        self.router = nn.Parameter(torch.empty(spec.experts, spec.dim))
        self.experts = nn.ModuleList([FeedForward(spec, spec.expert_hidden) for _ in range(spec.experts)])
        if spec.shared_expert_ff_dim:
            self.shared = FeedForward(spec, spec.shared_expert_ff_dim)
            self.shared_gate = nn.Parameter(torch.empty(1, spec.dim))
        else:
            self.shared = None
        self._stacked = None
        self._stack()

    def _apply(self, fn, *args, **kwargs):          # .to() / .cuda() / .bfloat16() give every parameter new storage
        out = super()._apply(fn, *args, **kwargs)
        self._stack()
        return out

    def _stack(self) -> None:
        ups, downs = [e.up_weight for e in self.experts], [e.down_weight for e in self.experts]
        self._stacked = None
        if any(e.up_bias is not None or e.down_bias is not None for e in self.experts):
            return
        if len({(p.dtype, p.device, tuple(p.shape)) for p in ups}) != 1 or ups[0].device.type == "meta":
            return
        with torch.no_grad():
            up, down = torch.stack([p.data for p in ups]), torch.stack([p.data for p in downs])
            for i, e in enumerate(self.experts):
                e.up_weight.data = up[i]
                e.down_weight.data = down[i]
        self._stacked = (up, down)

    def _stacked_now(self):
        """The stacked buffers when every expert's parameters still are their slices (something that re-homes
        parameters, a flat-bucket optimizer for one, ends that), else None."""
        if self._stacked is None:
            return None
        up, down = self._stacked
        for i, e in enumerate(self.experts):
            if (e.up_weight.data_ptr() != up[i].data_ptr() or e.down_weight.data_ptr() != down[i].data_ptr()
                    or getattr(e, "adapters", None) is not None or getattr(e, "packed", None)):
                return None
        return up, down

    def forward(self, x, residual=None):
        spec = self.spec
        from ..ops import moe
        kind = {"silu": "silu", "gelu": "gelu", "relu": "relu"}.get(spec.activation)
        st = self._stacked_now() if (x.is_cuda and kind is not None) else None
        if st is not None and moe.supported(x, st[0], st[1], spec.gated, kind):
            up = _AsStacked.apply(st[0], *[e.up_weight for e in self.experts])
            down = _AsStacked.apply(st[1], *[e.down_weight for e in self.experts])
            shared_res = residual
            if self.shared is not None:
                x2 = x.reshape(-1, x.shape[-1])
                g = torch.sigmoid((x2.float() * self.shared_gate.float()).sum(-1, keepdim=True)).to(x.dtype)
                sh = (self.shared(x2) * g).reshape(x.shape)
                shared_res = sh if residual is None else sh + residual
            return moe.routed_experts(x, self.router, up, down, spec.experts_per_token, spec.normalize_top_k,
                                      spec.gated, kind, shared_res)
        return self._forward_loop(x, residual)

    def _forward_loop(self, x, residual=None):
        """One pass per expert over the tokens that chose it: the host statement (and the path for shapes, adapters or
        packed weights the grouped kernels do not take)."""
        spec = self.spec
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = torch.nn.functional.linear(x2.float(), self.router.float())
        probs = torch.softmax(logits, -1)
        top_i = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, : spec.experts_per_token]
        top_p = probs.gather(1, top_i)
        if spec.normalize_top_k:
            top_p = top_p / top_p.sum(-1, keepdim=True)
        out = torch.zeros_like(x2, dtype=torch.float32)
        for e, expert in enumerate(self.experts):
            rows, slot = torch.nonzero(top_i == e, as_tuple=True)
            if rows.numel() == 0:
                continue
            y = expert(x2[rows])
            out.index_add_(0, rows, y.float() * top_p[rows, slot][:, None])
        if self.shared is not None:
            g = torch.sigmoid(torch.nn.functional.linear(x2.float(), self.shared_gate.float()))
            out = out + self.shared(x2).float() * g
        out = out.to(x.dtype).reshape(shape)
        return out + residual if residual is not None else out


class DecoderBlock(nn.Module):
    def __init__(self, spec: DecoderSpec, layer: int):
        super().__init__()
        self.spec, self.layer = spec, layer
        self.attn_norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.attn = SelfAttention(spec, layer)
        self.mlp_norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.mlp = MixtureOfExperts(spec) if spec.is_expert_layer(layer) else FeedForward(spec)
        if spec.post_norms:
            self.post_attn_norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
            self.post_mlp_norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.drop = spec.dropout

    def forward(self, x, positions=None, spans=None):
        spec = self.spec
        if spec.parallel_blocks:
            h = self.attn_norm(x)
            return x + self._drop(self.attn(h, None, positions, spans)) + self._drop(self.mlp(h))
        if spec.post_norms or self.drop > 0:
            a = self.attn(self.attn_norm(x), None, positions, spans)
            if spec.post_norms:
                a = self.post_attn_norm(a)
            x = x + self._drop(a)
            m = self.mlp(self.mlp_norm(x))
            if spec.post_norms:
                m = self.post_mlp_norm(m)
            return x + self._drop(m)
        # plain pre-norm block: residual additions happen inside the GEMM epilogues
        h, x = self.attn_norm.branch(x)
        x = self.attn(h, x, positions, spans)
        h, x = self.mlp_norm.branch(x)
        return self.mlp(h, x)

    def _drop(self, t):
        if self.drop > 0 and self.training:
            return torch.nn.functional.dropout(t, self.drop, True)
        return t


class Decoder(nn.Module):
    """Token embedding -> blocks -> final norm -> head. ``loss`` runs the head and the cross-entropy fused."""

    def __init__(self, spec: DecoderSpec):
        super().__init__()
        self.spec = spec
        vp = spec.padded_vocabulary
        self.embed = nn.Parameter(torch.empty(vp, spec.dim))
        self.pos = nn.Parameter(torch.empty(spec.max_positions, spec.dim)) if spec.learned_positions else None
        self.blocks = nn.ModuleList([DecoderBlock(spec, i) for i in range(spec.layers)])
        self.norm = Norm(spec.dim, spec.norm, spec.norm_epsilon, spec.norm_offset)
        self.head = None if spec.tie_embeddings else nn.Parameter(torch.empty(vp, spec.dim))
        self.head_bias = nn.Parameter(torch.zeros(vp)) if spec.head_bias else None
        if spec.tie_embeddings:
            self.embed._idrak_writers = 2      # its gradient comes from the head and from the lookup
        self.checkpoint_blocks = False
        self.loss_chunk_rows: Optional[int] = None
        self.reset_parameters()

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def reset_parameters(self, seed: Optional[int] = None):
        spec = self.spec
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        std = spec.init_std
        resid_std = std / math.sqrt(2 * spec.layers)

        def normal_(p, s):
            p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(s).to(p.dtype))

        normal_(self.embed, std)
        self.embed[spec.vocabulary:].zero_()
        if self.pos is not None:
            normal_(self.pos, std)
        if self.head is not None:
            normal_(self.head, std)
            self.head[spec.vocabulary:].zero_()
        for blk in self.blocks:
            normal_(blk.attn.qkv_weight, std)
            normal_(blk.attn.o_weight, resid_std)
            mlps = [blk.mlp] if isinstance(blk.mlp, FeedForward) else list(blk.mlp.experts) + (
                [blk.mlp.shared] if blk.mlp.shared is not None else [])
            for m in mlps:
                normal_(m.up_weight, std)
                normal_(m.down_weight, resid_std)
            if isinstance(blk.mlp, MixtureOfExperts):
                normal_(blk.mlp.router, std)
                if blk.mlp.shared is not None:
                    normal_(blk.mlp.shared_gate, std)

    # ------------------------------------------------------------------ forward
    def hidden(self, ids: torch.Tensor, positions: Optional[torch.Tensor] = None, spans=None,
               embeds=None) -> torch.Tensor:
        """Final hidden states. ``embeds``: ``(mask [B, S] bool, values [n, dim])`` - the rows of the token embedding at
        the masked positions are replaced by ``values`` in order (image or audio features projected into the model's
        width: the prefix a vision-language front end puts before the text)."""
        spec = self.spec
        B, S = ids.shape
        if self.pos is not None and positions is None:
            x = ops.embedding(ids, self.embed, self.pos)
        else:
            x = ops.embedding(ids, self.embed, None)
            if self.pos is not None:
                x = x + self.pos[positions.reshape(B, S).long()]
        if spec.embedding_scale is not None:
            x = x * spec.embedding_scale
        if embeds is not None:
            mask, values = embeds
            if int(mask.sum()) != values.shape[0]:
                raise ValueError(f"{int(mask.sum())} positions are marked for replacement but {values.shape[0]} rows were given")
            x = x.clone()
            x[mask] = values.to(x.dtype)
        if spec.dropout > 0 and self.training:
            x = torch.nn.functional.dropout(x, spec.dropout, True)
        if spans is not None and not torch.is_tensor(spans):
            spans = ops.row_starts_from_spans(spans, B, S, x.device)     # once per pass, not per layer
        for blk in self.blocks:
            if self.checkpoint_blocks and self.training and torch.is_grad_enabled():
                from ..core.checkpointing import checkpoint
                x = checkpoint(blk, x, positions, spans)
            else:
                x = blk(x, positions, spans)
        return self.norm(x)

    def head_weight(self) -> torch.Tensor:
        return self.embed if self.head is None else self.head

    def forward(self, ids: torch.Tensor, positions: Optional[torch.Tensor] = None, spans=None, embeds=None) -> torch.Tensor:
        """Logits ``[B, S, vocabulary]``. ``spans``: ``[(lo, hi), ...]`` token ranges of the sequences packed back to
        back into every row; attention stays inside each range (one kernel launch per layer: each position carries
        the start of its own sequence as a lower bound on the keys it sees)."""
        h = self.hidden(ids, positions, spans, embeds)
        logits = ops.linear(h, self.head_weight(), self.head_bias)[..., : self.spec.vocabulary]
        if self.spec.logit_softcap:
            c = self.spec.logit_softcap
            logits = torch.tanh(logits.float() / c).mul(c).to(logits.dtype)
        return logits

    def loss(self, ids: torch.Tensor, targets: torch.Tensor, positions: Optional[torch.Tensor] = None,
             ignore_index: Optional[int] = None, spans=None, embeds=None) -> torch.Tensor:
        """Mean next-token cross-entropy; the logits matrix is never materialised beyond one row chunk."""
        h = self.hidden(ids, positions, spans, embeds)
        if self.spec.logit_softcap or self.head_bias is not None:
            logits = self.forward_from_hidden(h)
            return torch.nn.functional.cross_entropy(
                logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1).long(),
                ignore_index=-100 if ignore_index is None else ignore_index)
        return ops.token_cross_entropy(h, self.head_weight(), targets, self.spec.vocabulary,
                                       self.loss_chunk_rows, ignore_index)

    def forward_from_hidden(self, h):
        logits = ops.linear(h, self.head_weight(), self.head_bias)[..., : self.spec.vocabulary]
        if self.spec.logit_softcap:
            c = self.spec.logit_softcap
            logits = torch.tanh(logits.float() / c).mul(c).to(logits.dtype)
        return logits

    # ------------------------------------------------------------------ parameter groups
    def decay_groups(self, weight_decay: float):
        """Matrices decay; biases, norms and 1-D tensors do not (the usual GPT recipe)."""
        decay, no_decay = [], []
        for _, p in self.named_parameters():
            (decay if p.dim() >= 2 else no_decay).append(p)
        return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


def build_decoder(spec: DecoderSpec, seed: Optional[int] = None) -> Decoder:
    model = Decoder(spec)
    if seed is not None:
        model.reset_parameters(seed)
    return model
