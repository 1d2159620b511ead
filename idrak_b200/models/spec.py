"""``DecoderSpec``: a decoder-only language model described as data.

Model families (Llama, Mistral, Qwen, Gemma, GPT-2 ...) are settings of this one record rather than
code; packages store it as JSON and checkpoints' configurations are translated into it.

Reference: DecoderSpec (src/Idrak.Abstraction/Generation/DecoderSpec.cs:62), RopeSettings /
RopeScalings (src/Idrak.Abstraction/Generation/RopeScalings.cs).
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field, fields
from typing import Optional, Sequence


@dataclass
class RopeSettings:
    """Rotary embedding: base, fraction of the head that rotates, and a context-extension scaling."""
    theta: float = 10000.0
    rotary_dim: Optional[int] = None          # None: the whole head
    scaling: Optional[str] = None             # None | "linear" | "dynamic" | "llama3" | "yarn"
    factor: float = 1.0
    original_max_positions: Optional[int] = None
    low_freq_factor: float = 1.0              # llama3
    high_freq_factor: float = 4.0             # llama3
    beta_fast: float = 32.0                   # yarn
    beta_slow: float = 1.0                    # yarn
    attention_factor: Optional[float] = None  # yarn

    def inv_freq(self, head_dim: int, seq_len: int | None = None):
        """Per-pair inverse frequencies (list of floats) after scaling, and the attention (mscale) factor."""
        rot = self.rotary_dim or head_dim
        half = rot // 2
        base = self.theta
        if self.scaling == "dynamic" and seq_len and self.original_max_positions and seq_len > self.original_max_positions:
            base = base * ((self.factor * seq_len / self.original_max_positions) - (self.factor - 1)) ** (rot / (rot - 2))
        inv = [base ** (-2.0 * k / rot) for k in range(half)]
        mscale = 1.0
        if self.scaling == "linear":
            inv = [f / self.factor for f in inv]
        elif self.scaling == "llama3":
            orig = self.original_max_positions or 8192
            low_wl, high_wl = orig / self.low_freq_factor, orig / self.high_freq_factor
            out = []
            for f in inv:
                wl = 2 * math.pi / f
                if wl < high_wl:
                    out.append(f)
                elif wl > low_wl:
                    out.append(f / self.factor)
                else:
                    smooth = (orig / wl - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
                    out.append((1 - smooth) * f / self.factor + smooth * f)
            inv = out
        elif self.scaling == "yarn":
            orig = self.original_max_positions or 4096

            def corr(n_rot):
                return (rot * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(self.theta))
            low = max(math.floor(corr(self.beta_fast)), 0)
            high = min(math.ceil(corr(self.beta_slow)), rot - 1)
            out = []
            for k, f in enumerate(inv):
                ramp = min(max((k - low) / max(high - low, 1e-3), 0.0), 1.0)
                extrap = 1.0 - ramp
                out.append(f / self.factor * (1 - extrap) + f * extrap)
            inv = out
            mscale = self.attention_factor if self.attention_factor is not None else (
                0.1 * math.log(self.factor) + 1.0 if self.factor > 1 else 1.0)
        return inv, mscale


@dataclass
class DecoderSpec:
    vocabulary: int
    dim: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    ff_dim: int
    max_positions: int
    norm: str = "rms"                          # "rms" | "layer"
    norm_epsilon: float = 1e-6
    norm_offset: float = 0.0                   # Gemma stores weight - 1
    gated: bool = True
    activation: str = "silu"                   # "silu" | "gelu" | "relu" | "tanh_sigmoid"
    rope: Optional[RopeSettings] = field(default_factory=RopeSettings)
    qkv_bias: bool = False
    output_bias: bool = False
    feed_forward_bias: bool = False
    qk_norm: bool = False
    post_norms: bool = False
    parallel_blocks: bool = False
    tie_embeddings: bool = False
    embedding_scale: Optional[float] = None
    head_bias: bool = False
    learned_positions: bool = False
    dropout: float = 0.0
    sliding_window: Optional[int] = None
    sliding_window_layers: Optional[Sequence[bool]] = None
    sliding_window_rope: Optional[RopeSettings] = None
    attention_scale: Optional[float] = None
    attention_softcap: Optional[float] = None
    logit_softcap: Optional[float] = None
    experts: int = 0
    experts_per_token: int = 0
    expert_ff_dim: int = 0
    shared_expert_ff_dim: int = 0
    normalize_top_k: bool = True
    expert_layers: Optional[Sequence[bool]] = None
    init_std: float = 0.02

    # ------------------------------------------------------------------ derived
    def is_expert_layer(self, layer: int) -> bool:
        return self.experts > 0 and (self.expert_layers is None or bool(self.expert_layers[layer]))

    def is_windowed(self, layer: int) -> bool:
        return self.sliding_window is not None and (
            self.sliding_window_layers is None or bool(self.sliding_window_layers[layer]))

    @property
    def expert_hidden(self) -> int:
        return self.expert_ff_dim if self.expert_ff_dim > 0 else self.ff_dim

    @property
    def padded_vocabulary(self) -> int:
        """Rows of the embedding / head tables: the vocabulary rounded up to a multiple of 64 so every row
        stride suits 16-byte vector access; rows beyond ``vocabulary`` never receive probability mass."""
        return (self.vocabulary + 63) // 64 * 64

    def _count(self, experts_counted: int) -> int:
        d, hd = self.dim, self.head_dim
        n = self.vocabulary * d
        if self.learned_positions:
            n += self.max_positions * d
        if not self.tie_embeddings:
            n += self.vocabulary * d + (self.vocabulary if self.head_bias else 0)
        norm_p = d * (2 if self.norm == "layer" else 1)
        for i in range(self.layers):
            n += norm_p * (2 + (2 if self.post_norms else 0))
            q, kv = self.heads * hd, self.kv_heads * hd
            n += d * (q + 2 * kv) + q * d
            if self.qkv_bias:
                n += q + 2 * kv
            if self.output_bias:
                n += d
            if self.qk_norm:
                n += 2 * hd
            mult = 3 if self.gated else 2
            if self.is_expert_layer(i):
                n += d * self.experts
                n += experts_counted * mult * d * self.expert_hidden
                if self.shared_expert_ff_dim:
                    n += mult * d * self.shared_expert_ff_dim + d
            else:
                n += mult * d * self.ff_dim
                if self.feed_forward_bias:
                    n += (2 if self.gated else 1) * self.ff_dim + d
        n += norm_p
        return n

    @property
    def parameter_count(self) -> int:
        return self._count(self.experts)

    @property
    def active_parameter_count(self) -> int:
        return self._count(self.experts_per_token)

    def flops_per_token(self, seq_len: int, training: bool = True) -> float:
        """Model FLOPs per token: 2 (6 with backward) per matmul weight + causal attention."""
        d = self.dim
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        per_layer = d * (q + 2 * kv) + q * d + (3 if self.gated else 2) * d * self.ff_dim
        mat = self.layers * per_layer + d * self.vocabulary
        attn = self.layers * 2 * self.heads * self.head_dim * seq_len / 2 * 2   # QK^T and PV, causal half
        f = 2.0 * (mat + attn)
        return f * 3 if training else f

    # ------------------------------------------------------------------ json
    def to_json(self) -> dict:
        d = asdict(self)
        return {k: v for k, v in d.items() if v is not None}

    def dumps(self) -> str:
        return json.dumps(self.to_json(), indent=2)

    @classmethod
    def from_json(cls, obj: dict | str) -> "DecoderSpec":
        if isinstance(obj, str):
            obj = json.loads(obj)
        known = {f.name for f in fields(cls)}
        unknown = set(obj) - known
        if unknown:
            raise ValueError(f"DecoderSpec: unknown keys {sorted(unknown)}")
        kw = dict(obj)
        for key in ("rope", "sliding_window_rope"):
            if isinstance(kw.get(key), dict):
                kw[key] = RopeSettings(**kw[key])
        if "rope" not in obj:
            kw["rope"] = None
        return cls(**kw)

    # ------------------------------------------------------------------ presets
    @classmethod
    def gpt2(cls, layers=12, dim=768, heads=12, vocab=50257, max_positions=1024, ff_dim=None, dropout=0.0):
        """GPT-2 style: LayerNorm, learned positions, plain GELU-tanh MLP with biases, tied head."""
        return cls(vocabulary=vocab, dim=dim, layers=layers, heads=heads, kv_heads=heads, head_dim=dim // heads,
                   ff_dim=ff_dim or 4 * dim, max_positions=max_positions, norm="layer", norm_epsilon=1e-5,
                   gated=False, activation="gelu", rope=None, qkv_bias=True, output_bias=True,
                   feed_forward_bias=True, tie_embeddings=True, learned_positions=True, dropout=dropout)

    @classmethod
    def llama(cls, layers=32, dim=4096, heads=32, kv_heads=8, ff_dim=14336, vocab=128256, max_positions=8192,
              theta=500000.0, eps=1e-5, head_dim=None, tie=False):
        """Llama style: RMSNorm, RoPE, grouped-query attention, SwiGLU, no biases."""
        return cls(vocabulary=vocab, dim=dim, layers=layers, heads=heads, kv_heads=kv_heads,
                   head_dim=head_dim or dim // heads, ff_dim=ff_dim, max_positions=max_positions, norm="rms",
                   norm_epsilon=eps, gated=True, activation="silu", rope=RopeSettings(theta=theta),
                   tie_embeddings=tie)

    @classmethod
    def tiny_gpt(cls):
        """The small CPU sample: 4 layers, d_model 128, 4 heads, MLP 512 GELU, byte vocabulary, 128 positions."""
        return cls.gpt2(layers=4, dim=128, heads=4, vocab=256, max_positions=128)
