"""Encoder families: BERT-style bidirectional encoders (sentence embeddings, cross-encoder scoring, masked-token
heads) and T5 encoder-decoders (relative position buckets, unscaled attention, gated or plain feed-forward) with a
greedy / sampled sequence-to-sequence generator. Both load Hugging Face tensor names.

Projections go through ``ops.linear`` (the tcgen05 GEMM on bf16 CUDA tensors), norms through ``ops.layer_norm`` /
``ops.rms_norm``; attention with padding masks or position biases uses the library's fused attention.

Reference: the BERT and T5 families of src/Idrak.Text.Plugins, ``EncoderModels`` (src/Idrak/Models), cross-encoder
reranking in the retrieval package and ``Seq2SeqGenerator`` (src/Idrak/Generation).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops


def _linear(x, w, b=None, residual=None):
    if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[1] % 8 == 0:
        return ops.linear(x, w, b, residual)
    y = F.linear(x, w, b)
    return y if residual is None else y + residual


# ---------------------------------------------------------------------------------------------------------------------
# BERT
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class BertSpec:
    vocab: int = 30522
    dim: int = 768
    layers: int = 12
    heads: int = 12
    ff_dim: int = 3072
    max_positions: int = 512
    type_vocab: int = 2
    norm_epsilon: float = 1e-12
    labels: int = 0                      # > 0: a sequence-classification head (cross-encoder: 1)

    @classmethod
    def from_hf_config(cls, c: dict) -> "BertSpec":
        return cls(c["vocab_size"], c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"], c["intermediate_size"],
                   c.get("max_position_embeddings", 512), c.get("type_vocab_size", 2), c.get("layer_norm_eps", 1e-12),
                   len(c.get("id2label", {})) if "id2label" in c else c.get("num_labels", 0))


class BertLayer(nn.Module):
    def __init__(self, s: BertSpec):
        super().__init__()
        self.s = s
        d = s.dim
        self.qkv_w, self.qkv_b = nn.Parameter(torch.empty(3 * d, d)), nn.Parameter(torch.zeros(3 * d))
        self.o_w, self.o_b = nn.Parameter(torch.empty(d, d)), nn.Parameter(torch.zeros(d))
        self.norm1_w, self.norm1_b = nn.Parameter(torch.ones(d)), nn.Parameter(torch.zeros(d))
        self.up_w, self.up_b = nn.Parameter(torch.empty(s.ff_dim, d)), nn.Parameter(torch.zeros(s.ff_dim))
        self.down_w, self.down_b = nn.Parameter(torch.empty(d, s.ff_dim)), nn.Parameter(torch.zeros(d))
        self.norm2_w, self.norm2_b = nn.Parameter(torch.ones(d)), nn.Parameter(torch.zeros(d))

    def forward(self, x, mask):
        s = self.s
        N, T, C = x.shape
        D = C // s.heads
        q, k, v = _linear(x, self.qkv_w, self.qkv_b).view(N, T, 3, s.heads, D).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(N, T, C)
        x = F.layer_norm(_linear(a, self.o_w, self.o_b, x), (C,), self.norm1_w, self.norm1_b, s.norm_epsilon)   # post-norm
        h = F.gelu(_linear(x, self.up_w, self.up_b))
        return F.layer_norm(_linear(h, self.down_w, self.down_b, x), (C,), self.norm2_w, self.norm2_b, s.norm_epsilon)


class BertEncoder(nn.Module):
    def __init__(self, spec: BertSpec):
        super().__init__()
        self.spec = s = spec
        self.word = nn.Parameter(torch.empty(s.vocab, s.dim))
        self.position = nn.Parameter(torch.empty(s.max_positions, s.dim))
        self.token_type = nn.Parameter(torch.empty(s.type_vocab, s.dim))
        self.embed_norm_w, self.embed_norm_b = nn.Parameter(torch.ones(s.dim)), nn.Parameter(torch.zeros(s.dim))
        self.layers = nn.ModuleList([BertLayer(s) for _ in range(s.layers)])
        self.pool_w, self.pool_b = nn.Parameter(torch.empty(s.dim, s.dim)), nn.Parameter(torch.zeros(s.dim))
        if s.labels:
            self.class_w, self.class_b = nn.Parameter(torch.empty(s.labels, s.dim)), nn.Parameter(torch.zeros(s.labels))
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.normal_(0, 0.02)

    def hidden(self, ids, attention_mask=None, token_types=None):
        s = self.spec
        N, T = ids.shape
        if T > s.max_positions:
            raise ValueError(f"{T} tokens; the model has {s.max_positions} positions")
        types = token_types if token_types is not None else torch.zeros_like(ids)
        x = self.word[ids.long()] + self.position[:T][None] + self.token_type[types.long()]
        x = F.layer_norm(x, (s.dim,), self.embed_norm_w, self.embed_norm_b, s.norm_epsilon)
        mask = None
        if attention_mask is not None:
            mask = attention_mask.bool()[:, None, None, :]
        for layer in self.layers:
            x = layer(x, mask)
        return x

    def pooled(self, ids, attention_mask=None, token_types=None):
        """tanh(W h[CLS] + b): the library's pooled output."""
        h = self.hidden(ids, attention_mask, token_types)
        return torch.tanh(_linear(h[:, 0].contiguous(), self.pool_w, self.pool_b))

    def embed(self, ids, attention_mask=None, pooling: str = "mean"):
        """Unit-length sentence vectors: mean over real tokens, or the first token."""
        h = self.hidden(ids, attention_mask).float()
        if pooling == "cls":
            v = h[:, 0]
        else:
            m = (attention_mask if attention_mask is not None else torch.ones_like(ids)).float()[..., None]
            v = (h * m).sum(1) / m.sum(1).clamp_min(1.0)
        return F.normalize(v, dim=-1)

    def classify(self, ids, attention_mask=None, token_types=None):
        """Logits of the classification head over the pooled output (a cross-encoder's relevance score)."""
        if not self.spec.labels:
            raise ValueError("this encoder has no classification head")
        return _linear(self.pooled(ids, attention_mask, token_types), self.class_w, self.class_b)

    def load_hf_tensors(self, src: Mapping[str, torch.Tensor]) -> None:
        def get(name):
            for prefix in ("bert.", ""):
                if prefix + name in src:
                    return src[prefix + name]
            raise KeyError(f"the checkpoint has no tensor '{name}'")
        with torch.no_grad():
            self.word.copy_(get("embeddings.word_embeddings.weight"))
            self.position.copy_(get("embeddings.position_embeddings.weight"))
            self.token_type.copy_(get("embeddings.token_type_embeddings.weight"))
            self.embed_norm_w.copy_(get("embeddings.LayerNorm.weight")); self.embed_norm_b.copy_(get("embeddings.LayerNorm.bias"))
            for i, l in enumerate(self.layers):
                p = f"encoder.layer.{i}."
                l.qkv_w.copy_(torch.cat([get(p + f"attention.self.{n}.weight") for n in ("query", "key", "value")]))
                l.qkv_b.copy_(torch.cat([get(p + f"attention.self.{n}.bias") for n in ("query", "key", "value")]))
                l.o_w.copy_(get(p + "attention.output.dense.weight")); l.o_b.copy_(get(p + "attention.output.dense.bias"))
                l.norm1_w.copy_(get(p + "attention.output.LayerNorm.weight")); l.norm1_b.copy_(get(p + "attention.output.LayerNorm.bias"))
                l.up_w.copy_(get(p + "intermediate.dense.weight")); l.up_b.copy_(get(p + "intermediate.dense.bias"))
                l.down_w.copy_(get(p + "output.dense.weight")); l.down_b.copy_(get(p + "output.dense.bias"))
                l.norm2_w.copy_(get(p + "output.LayerNorm.weight")); l.norm2_b.copy_(get(p + "output.LayerNorm.bias"))
            if "bert.pooler.dense.weight" in src or "pooler.dense.weight" in src:
                self.pool_w.copy_(get("pooler.dense.weight")); self.pool_b.copy_(get("pooler.dense.bias"))
            if self.spec.labels and "classifier.weight" in src:
                self.class_w.copy_(src["classifier.weight"]); self.class_b.copy_(src["classifier.bias"])


# ---------------------------------------------------------------------------------------------------------------------
# T5
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class T5Spec:
    vocab: int = 32128
    dim: int = 512
    layers: int = 6
    decoder_layers: int = 6
    heads: int = 8
    head_dim: int = 64
    ff_dim: int = 2048
    buckets: int = 32
    max_distance: int = 128
    gated: bool = False                  # v1.1: gated GELU feed-forward and an untied output head
    tied_head: bool = True
    norm_epsilon: float = 1e-6
    pad_id: int = 0
    eos_id: int = 1
    start_id: int = 0

    @classmethod
    def from_hf_config(cls, c: dict) -> "T5Spec":
        gated = "gated" in c.get("feed_forward_proj", "relu")
        return cls(c["vocab_size"], c["d_model"], c["num_layers"], c.get("num_decoder_layers", c["num_layers"]), c["num_heads"],
                   c["d_kv"], c["d_ff"], c.get("relative_attention_num_buckets", 32), c.get("relative_attention_max_distance", 128),
                   gated, c.get("tie_word_embeddings", True), c.get("layer_norm_epsilon", 1e-6), c.get("pad_token_id", 0),
                   c.get("eos_token_id", 1), c.get("decoder_start_token_id", 0))


def relative_buckets(relative: torch.Tensor, bidirectional: bool, buckets: int, max_distance: int) -> torch.Tensor:
    """T5's position buckets: half exact small offsets, half logarithmic up to ``max_distance``; the encoder splits
    the buckets between the two directions."""
    ret = torch.zeros_like(relative)
    n = buckets
    if bidirectional:
        n //= 2
        ret = ret + (relative > 0).long() * n
        rel = relative.abs()
    else:
        rel = -torch.minimum(relative, torch.zeros_like(relative))
    exact = n // 2
    large = exact + (torch.log(rel.float().clamp_min(1) / exact) / math.log(max_distance / exact) * (n - exact)).long()
    large = torch.minimum(large, torch.full_like(large, n - 1))
    return ret + torch.where(rel < exact, rel, large)


class T5Attention(nn.Module):
    def __init__(self, s: T5Spec, bias_table: bool, bidirectional: bool):
        super().__init__()
        self.s, self.bidirectional = s, bidirectional
        inner = s.heads * s.head_dim
        self.q, self.k = nn.Parameter(torch.empty(inner, s.dim)), nn.Parameter(torch.empty(inner, s.dim))
        self.v, self.o = nn.Parameter(torch.empty(inner, s.dim)), nn.Parameter(torch.empty(s.dim, inner))
        self.bias = nn.Parameter(torch.empty(s.buckets, s.heads)) if bias_table else None

    def position_bias(self, q_len: int, k_len: int, device, offset: int = 0) -> torch.Tensor:
        ctx = torch.arange(offset, offset + q_len, device=device)[:, None]
        mem = torch.arange(k_len, device=device)[None]
        b = relative_buckets(mem - ctx, self.bidirectional, self.s.buckets, self.s.max_distance)
        return self.bias[b].permute(2, 0, 1)[None]                   # [1, heads, q, k]

    def forward(self, x, memory, bias, residual):
        s = self.s
        N, T, _ = x.shape
        S = memory.shape[1]
        q = _linear(x, self.q).view(N, T, s.heads, s.head_dim).transpose(1, 2)
        k = _linear(memory, self.k).view(N, S, s.heads, s.head_dim).transpose(1, 2)
        v = _linear(memory, self.v).view(N, S, s.heads, s.head_dim).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype) if bias is not None else None, scale=1.0)
        return _linear(a.transpose(1, 2).reshape(N, T, -1), self.o, None, residual)


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class T5Block(nn.Module):
    def __init__(self, s: T5Spec, decoder: bool, first: bool):
        super().__init__()
        self.s, self.decoder = s, decoder
        self.self_norm = nn.Parameter(torch.ones(s.dim))
        self.self_attn = T5Attention(s, bias_table=first, bidirectional=not decoder)
        if decoder:
            self.cross_norm = nn.Parameter(torch.ones(s.dim))
            self.cross_attn = T5Attention(s, bias_table=False, bidirectional=False)
        self.ff_norm = nn.Parameter(torch.ones(s.dim))
        self.wi = nn.Parameter(torch.empty((2 if s.gated else 1) * s.ff_dim, s.dim))
        self.wo = nn.Parameter(torch.empty(s.dim, s.ff_dim))

    def forward(self, x, self_bias, memory=None, cross_bias=None):
        s = self.s
        h = _rms(x, self.self_norm, s.norm_epsilon)
        x = self.self_attn(h, h, self_bias, x)
        if self.decoder:
            x = self.cross_attn(_rms(x, self.cross_norm, s.norm_epsilon), memory, cross_bias, x)
        h = _linear(_rms(x, self.ff_norm, s.norm_epsilon), self.wi)
        if s.gated:
            g, u = h.split(s.ff_dim, -1)
            h = F.gelu(g, approximate="tanh") * u
        else:
            h = F.relu(h)
        return _linear(h, self.wo, None, x)


class T5(nn.Module):
    def __init__(self, spec: T5Spec):
        super().__init__()
        self.spec = s = spec
        self.shared = nn.Parameter(torch.empty(s.vocab, s.dim))
        self.encoder = nn.ModuleList([T5Block(s, False, i == 0) for i in range(s.layers)])
        self.decoder = nn.ModuleList([T5Block(s, True, i == 0) for i in range(s.decoder_layers)])
        self.encoder_norm, self.decoder_norm = nn.Parameter(torch.ones(s.dim)), nn.Parameter(torch.ones(s.dim))
        self.head = None if s.tied_head else nn.Parameter(torch.empty(s.vocab, s.dim))
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.normal_(0, 0.05)

    def encode(self, ids, attention_mask=None):
        s = self.spec
        x = self.shared[ids.long()]
        T = ids.shape[1]
        bias = self.encoder[0].self_attn.position_bias(T, T, ids.device).float()
        if attention_mask is not None:
            bias = bias + (1.0 - attention_mask.float())[:, None, None, :] * torch.finfo(torch.float32).min
        for b in self.encoder:
            x = b(x, bias)
        return _rms(x, self.encoder_norm, s.norm_epsilon)

    def decode(self, decoder_ids, memory, memory_mask=None):
        """Logits ``[N, T, vocab]`` for the decoder inputs given the encoder output."""
        s = self.spec
        x = self.shared[decoder_ids.long()]
        T = decoder_ids.shape[1]
        bias = self.decoder[0].self_attn.position_bias(T, T, x.device).float()
        causal = torch.full((T, T), torch.finfo(torch.float32).min, device=x.device).triu(1)
        bias = bias + causal[None, None]
        cross = None
        if memory_mask is not None:
            cross = (1.0 - memory_mask.float())[:, None, None, :] * torch.finfo(torch.float32).min
        for b in self.decoder:
            x = b(x, bias, memory, cross)
        x = _rms(x, self.decoder_norm, s.norm_epsilon)
        if s.tied_head:
            return _linear(x * (s.dim ** -0.5), self.shared)
        return _linear(x, self.head)

    def forward(self, ids, decoder_ids, attention_mask=None):
        return self.decode(decoder_ids, self.encode(ids, attention_mask), attention_mask)

    def loss(self, ids, labels, attention_mask=None):
        """Teacher forcing: decoder inputs are the labels shifted right behind the start token; -100 labels are ignored."""
        s = self.spec
        start = torch.full_like(labels[:, :1], s.start_id)
        dec = torch.cat([start, labels[:, :-1].clamp_min(0)], 1)
        logits = self.forward(ids, dec, attention_mask)
        return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1).long(), ignore_index=-100)

    def load_hf_tensors(self, src: Mapping[str, torch.Tensor]) -> None:
        s = self.spec
        with torch.no_grad():
            self.shared.copy_(src["shared.weight"])
            for side, blocks in (("encoder", self.encoder), ("decoder", self.decoder)):
                for i, b in enumerate(blocks):
                    p = f"{side}.block.{i}.layer."
                    a = p + "0.SelfAttention."
                    for n in ("q", "k", "v", "o"):
                        getattr(b.self_attn, n).copy_(src[a + f"{n}.weight"])
                    if b.self_attn.bias is not None:
                        b.self_attn.bias.copy_(src[a + "relative_attention_bias.weight"])
                    b.self_norm.copy_(src[p + "0.layer_norm.weight"])
                    ff = 1
                    if side == "decoder":
                        c = p + "1.EncDecAttention."
                        for n in ("q", "k", "v", "o"):
                            getattr(b.cross_attn, n).copy_(src[c + f"{n}.weight"])
                        b.cross_norm.copy_(src[p + "1.layer_norm.weight"])
                        ff = 2
                    d = p + f"{ff}.DenseReluDense."
                    if s.gated:
                        b.wi.copy_(torch.cat([src[d + "wi_0.weight"], src[d + "wi_1.weight"]]))
                    else:
                        b.wi.copy_(src[d + "wi.weight"])
                    b.wo.copy_(src[d + "wo.weight"])
                    b.ff_norm.copy_(src[p + f"{ff}.layer_norm.weight"])
            self.encoder_norm.copy_(src["encoder.final_layer_norm.weight"])
            self.decoder_norm.copy_(src["decoder.final_layer_norm.weight"])
            if self.head is not None:
                self.head.copy_(src["lm_head.weight"])


class Seq2SeqGenerator:
    """Encode once, then decode token by token (greedy, or sampled with a temperature and top-k) until the
    end-of-sequence token or ``max_tokens``. The decoder re-reads its prefix each step (prefixes here are short)."""

    def __init__(self, model: T5):
        self.model = model.eval()

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, max_tokens: int = 64,
                 temperature: float = 0.0, top_k: int = 0, seed: int = 0) -> List[List[int]]:
        s = self.model.spec
        memory = self.model.encode(ids, attention_mask)
        N = ids.shape[0]
        out = torch.full((N, 1), s.start_id, dtype=torch.long, device=ids.device)
        done = torch.zeros(N, dtype=torch.bool, device=ids.device)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for _ in range(max_tokens):
            logits = self.model.decode(out, memory, attention_mask)[:, -1].float()
            if temperature > 0:
                logits = logits / temperature
                if top_k:
                    kth = logits.topk(top_k).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                nxt = torch.multinomial(logits.softmax(-1).cpu(), 1, generator=gen)[:, 0].to(ids.device)
            else:
                nxt = logits.argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, s.pad_id), nxt)
            out = torch.cat([out, nxt[:, None]], 1)
            done |= nxt == s.eos_id
            if bool(done.all()):
                break
        rows = []
        for r in out[:, 1:].tolist():
            rows.append(r[: r.index(s.eos_id)] if s.eos_id in r else [t for t in r if t != s.pad_id or s.pad_id == s.start_id])
        return rows
