"""Whisper: an audio encoder (two 1-D convolutions over the log-mel spectrogram, sinusoidal positions, pre-norm
transformer layers) and a text decoder with cross-attention, in the Hugging Face weight layout.

``WhisperSpec.from_hf_config`` reads ``config.json``; ``Whisper.load_hf`` takes the checkpoint's tensors by their
Hugging Face names; ``features`` turns 16 kHz samples into the model's input (30 s windows of 80 or 128 mel bands,
log10, clamped to 8 decades below the peak, scaled to about [-1, 1]); ``generate`` decodes greedily with a key / value
cache (the cross-attention keys and values of the audio are computed once), starting from the forced prefix
(start-of-transcript, language, task, no-timestamps) the caller gives.

Reference: the Whisper speech family (samples/WhisperSpeech, src/Idrak.Audio speech models) - encoder / decoder layout
and feature extraction follow the published model so that its checkpoints load unchanged.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from . import MelSpec, log_mel


@dataclass
class WhisperSpec:
    mels: int = 80
    vocabulary: int = 51865
    dim: int = 384
    encoder_layers: int = 4
    decoder_layers: int = 4
    heads: int = 6
    ff_dim: int = 1536
    source_positions: int = 1500
    target_positions: int = 448

    @classmethod
    def from_hf_config(cls, c: dict) -> "WhisperSpec":
        return cls(c["num_mel_bins"], c["vocab_size"], c["d_model"], c["encoder_layers"], c["decoder_layers"],
                   c["encoder_attention_heads"], c["encoder_ffn_dim"], c["max_source_positions"], c["max_target_positions"])


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """The encoder's fixed position table: sines in the first half of the channels, cosines in the second."""
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], 1)


class _Attention(nn.Module):
    """Multi-head attention with the checkpoint's bias pattern (no bias on the key projection)."""

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.q, self.k = nn.Linear(dim, dim), nn.Linear(dim, dim, bias=False)
        self.v, self.out = nn.Linear(dim, dim), nn.Linear(dim, dim)

    def _split(self, t):
        n, s, c = t.shape
        return t.view(n, s, self.heads, c // self.heads).transpose(1, 2)

    def keys_values(self, memory):
        return self._split(self.k(memory)), self._split(self.v(memory))

    def forward(self, x, memory=None, causal: bool = False, cache: Optional[dict] = None, fixed: Optional[tuple] = None):
        q = self._split(self.q(x))
        if fixed is not None:                               # cross-attention over keys / values computed once
            k, v = fixed
        else:
            k, v = self.keys_values(x if memory is None else memory)
            if cache is not None:                           # self-attention while decoding: append to what is kept
                if "k" in cache:
                    k, v = torch.cat([cache["k"], k], 2), torch.cat([cache["v"], v], 2)
                cache["k"], cache["v"] = k, v
        a = F.scaled_dot_product_attention(q, k, v, is_causal=causal and q.shape[2] > 1 and q.shape[2] == k.shape[2])
        n, _, s, _ = a.shape
        return self.out(a.transpose(1, 2).reshape(n, s, -1))


class _Layer(nn.Module):
    def __init__(self, dim: int, heads: int, ff_dim: int, cross: bool):
        super().__init__()
        self.self_norm, self.self_attn = nn.LayerNorm(dim), _Attention(dim, heads)
        self.cross_norm = nn.LayerNorm(dim) if cross else None
        self.cross_attn = _Attention(dim, heads) if cross else None
        self.ff_norm, self.fc1, self.fc2 = nn.LayerNorm(dim), nn.Linear(dim, ff_dim), nn.Linear(ff_dim, dim)

    def forward(self, x, causal=False, cache=None, cross=None):
        x = x + self.self_attn(self.self_norm(x), causal=causal, cache=cache)
        if self.cross_attn is not None:
            x = x + self.cross_attn(self.cross_norm(x), fixed=cross)
        return x + self.fc2(F.gelu(self.fc1(self.ff_norm(x))))


class Whisper(nn.Module):
    def __init__(self, spec: WhisperSpec):
        super().__init__()
        s = self.spec = spec
        self.conv1 = nn.Conv1d(s.mels, s.dim, 3, padding=1)
        self.conv2 = nn.Conv1d(s.dim, s.dim, 3, stride=2, padding=1)
        self.register_buffer("source_positions", sinusoids(s.source_positions, s.dim))
        self.encoder = nn.ModuleList(_Layer(s.dim, s.heads, s.ff_dim, False) for _ in range(s.encoder_layers))
        self.encoder_norm = nn.LayerNorm(s.dim)
        self.tokens = nn.Embedding(s.vocabulary, s.dim)
        self.target_positions = nn.Embedding(s.target_positions, s.dim)
        self.decoder = nn.ModuleList(_Layer(s.dim, s.heads, s.ff_dim, True) for _ in range(s.decoder_layers))
        self.decoder_norm = nn.LayerNorm(s.dim)

    # ------------------------------------------------------------------ the two halves
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """``mel`` ``[N, mels, frames]`` (frames = 2 x source positions) -> ``[N, source positions, dim]``."""
        x = F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)
        x = x + self.source_positions[: x.shape[1]].to(x.dtype)
        for layer in self.encoder:
            x = layer(x)
        return self.encoder_norm(x)

    def cross_keys_values(self, audio: torch.Tensor):
        return [layer.cross_attn.keys_values(audio) for layer in self.decoder]

    def decode(self, ids: torch.Tensor, cross, caches: Optional[List[dict]] = None, offset: int = 0) -> torch.Tensor:
        """Logits ``[N, T, vocabulary]`` for ``ids`` ``[N, T]`` at positions ``offset ..``; ``cross`` from
        ``cross_keys_values``; ``caches`` (one dict per layer) makes the call incremental."""
        pos = torch.arange(offset, offset + ids.shape[1], device=ids.device)
        x = self.tokens(ids) + self.target_positions(pos)
        for i, layer in enumerate(self.decoder):
            x = layer(x, causal=True, cache=None if caches is None else caches[i], cross=cross[i])
        return self.decoder_norm(x) @ self.tokens.weight.t()

    def forward(self, mel: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        return self.decode(ids, self.cross_keys_values(self.encode(mel)))

    @torch.no_grad()
    def generate(self, mel: torch.Tensor, prefix: Sequence[int], end_token: int, max_tokens: int = 224,
                 suppress: Sequence[int] = ()) -> List[List[int]]:
        """Greedy transcription token ids (without the prefix) for each spectrogram of the batch."""
        n = mel.shape[0]
        cross = self.cross_keys_values(self.encode(mel))
        caches = [dict() for _ in self.decoder]
        ids = torch.tensor([list(prefix)] * n, device=mel.device)
        logits = self.decode(ids, cross, caches)[:, -1]
        out: List[List[int]] = [[] for _ in range(n)]
        done = torch.zeros(n, dtype=torch.bool, device=mel.device)
        offset = ids.shape[1]
        limit = min(max_tokens, self.spec.target_positions - offset)
        for _ in range(limit):
            if suppress:
                logits[:, list(suppress)] = float("-inf")
            nxt = logits.float().argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, end_token), nxt)
            for i, t in enumerate(nxt.tolist()):
                if not done[i] and t != end_token:
                    out[i].append(t)
            done = done | (nxt == end_token)
            if bool(done.all()):
                break
            logits = self.decode(nxt[:, None], cross, caches, offset)[:, -1]
            offset += 1
        return out

    # ------------------------------------------------------------------ checkpoints
    def load_hf(self, tensors: Dict[str, torch.Tensor]) -> List[str]:
        """Copy a Hugging Face checkpoint in; returns the names it did not find (empty for a complete checkpoint)."""
        t = {k[len("model."):] if k.startswith("model.") else k: v for k, v in tensors.items()}
        missing: List[str] = []

        def put(param, name):
            if name in t:
                with torch.no_grad():
                    param.copy_(t[name].to(param.dtype))
            else:
                missing.append(name)

        def attention(a: _Attention, prefix):
            for mine, theirs in ((a.q, "q_proj"), (a.k, "k_proj"), (a.v, "v_proj"), (a.out, "out_proj")):
                put(mine.weight, f"{prefix}.{theirs}.weight")
                if mine.bias is not None:
                    put(mine.bias, f"{prefix}.{theirs}.bias")

        def norm(nrm, prefix):
            put(nrm.weight, prefix + ".weight")
            put(nrm.bias, prefix + ".bias")

        for side, layers in (("encoder", self.encoder), ("decoder", self.decoder)):
            for i, layer in enumerate(layers):
                p = f"{side}.layers.{i}"
                attention(layer.self_attn, p + ".self_attn")
                norm(layer.self_norm, p + ".self_attn_layer_norm")
                if layer.cross_attn is not None:
                    attention(layer.cross_attn, p + ".encoder_attn")
                    norm(layer.cross_norm, p + ".encoder_attn_layer_norm")
                put(layer.fc1.weight, p + ".fc1.weight"); put(layer.fc1.bias, p + ".fc1.bias")
                put(layer.fc2.weight, p + ".fc2.weight"); put(layer.fc2.bias, p + ".fc2.bias")
                norm(layer.ff_norm, p + ".final_layer_norm")
        for conv, name in ((self.conv1, "encoder.conv1"), (self.conv2, "encoder.conv2")):
            put(conv.weight, name + ".weight")
            put(conv.bias, name + ".bias")
        if "encoder.embed_positions.weight" in t:
            self.source_positions.copy_(t["encoder.embed_positions.weight"].to(self.source_positions.dtype))
        norm(self.encoder_norm, "encoder.layer_norm")
        put(self.tokens.weight, "decoder.embed_tokens.weight")
        put(self.target_positions.weight, "decoder.embed_positions.weight")
        norm(self.decoder_norm, "decoder.layer_norm")
        return missing


def features(samples: torch.Tensor, mels: int = 80, rate: int = 16000, seconds: int = 30) -> torch.Tensor:
    """Model input ``[mels, seconds * 100]`` from mono samples at ``rate`` Hz: padded or cut to the window, 25 ms
    frames every 10 ms, log10 of the mel power clamped to 8 decades below the peak, then ``(x + 4) / 4``
    (``audio.log_mel`` with ``MelSpec.whisper``)."""
    if rate != 16000:
        from . import resample
        samples = resample(samples.float().reshape(-1), rate, 16000)
    n = 16000 * seconds
    x = samples.float().reshape(-1)[:n]
    x = F.pad(x, (0, n - x.numel()))
    return log_mel(x, MelSpec.whisper(mels))
