"""VITS text-to-speech: a conditional variational autoencoder with a normalising-flow prior, a HiFi-GAN waveform
generator and a duration model, for synthesis and for (adversarial) training.

Parts, all channels-first ``[B, C, T]``:

* ``TextEncoder``: token embedding, post-norm Transformer layers whose attention adds learned key / value vectors for
  relative offsets inside a window, convolutional feed-forward, and a projection to the prior's mean and log-deviation
  per token;
* ``WaveNet``: gated dilated convolutions with skip sums and an optional global (speaker) condition; it is the body of
  the ``PosteriorEncoder`` (linear spectrogram -> latent) and of every mean-only ``Coupling`` of the ``Flow``;
* ``DurationPredictor``: two normalised convolutions -> log-frames per token;
* ``Generator``: HiFi-GAN (transposed-convolution up-sampling, multi-receptive-field residual blocks);
* ``monotonic_alignment``: the most likely monotonic, surjective alignment of spectrogram frames to tokens under the
  prior (dynamic programme over the frames, batched over sequences and tokens);
* ``Vits.synthesize`` (text -> waveform) and ``Vits.training_losses`` (alignment, duration loss, KL divergence between
  posterior and flowed prior, generated segment for the spectral and adversarial losses);
* ``Vits.convert_voice`` (a recording re-voiced through the flow under another speaker) with ``ReferenceEncoder``
  (a speaker embedding from any recording's spectrogram: the tone-colour half of voice cloning);
* ``Discriminators`` (multi-period + one multi-scale branch) with the least-squares adversarial and feature-matching
  losses.

Weights load from the Hugging Face ``VitsModel`` layout (weight-normalised convolutions are folded on load); with the
sampling noise off, ``synthesize`` reproduces that implementation's waveform (``tests/test_vits.py``), with either
duration model: the deterministic ``DurationPredictor`` or the ``StochasticDurationPredictor`` (a spline flow sampled
backwards for synthesis and trained forwards by a variational bound) that the published checkpoints use.
On CUDA the 1-D convolutions run on this package's convolution kernels (``nn/layers.py: Conv1d``).

Reference: the speech trainer's TTS / adversarial VITS modes and the VITS plugin (src/Idrak.Audio, src/Idrak.Plugins).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.layers import Conv1d


@dataclass
class VitsSpec:
    vocab_size: int = 38
    hidden: int = 192
    layers: int = 6
    heads: int = 2
    window: int = 4
    ffn: int = 768
    ffn_kernel: int = 3
    flow_size: int = 192
    spectrogram_bins: int = 513
    duration_filter: int = 256
    duration_kernel: int = 3
    prior_flows: int = 4
    prior_wavenet_layers: int = 4
    posterior_wavenet_layers: int = 16
    wavenet_kernel: int = 5
    wavenet_dilation: int = 1
    upsample_rates: Tuple[int, ...] = (8, 8, 2, 2)
    upsample_kernels: Tuple[int, ...] = (16, 16, 4, 4)
    upsample_channels: int = 512
    resblock_kernels: Tuple[int, ...] = (3, 7, 11)
    resblock_dilations: Tuple[Tuple[int, ...], ...] = ((1, 3, 5), (1, 3, 5), (1, 3, 5))
    leaky_slope: float = 0.1
    speakers: int = 1
    speaker_dim: int = 0
    eps: float = 1e-5
    noise_scale: float = 0.667
    speaking_rate: float = 1.0
    sampling_rate: int = 16000
    bias: bool = True
    stochastic_duration: bool = False
    duration_flows: int = 4
    duration_flow_bins: int = 10
    duration_tail_bound: float = 5.0
    duration_stack_layers: int = 3
    duration_dropout: float = 0.5
    noise_scale_duration: float = 0.8

    @property
    def hop(self) -> int:
        return int(math.prod(self.upsample_rates))

    @classmethod
    def from_hf(cls, c: Dict) -> "VitsSpec":
        """From the keys of a Hugging Face ``VitsConfig`` (a dict, e.g. the parsed ``config.json``)."""
        g = c.get
        if g("depth_separable_channels", 2) != 2:
            raise ValueError("the stochastic duration predictor here carries two channels (duration and its companion)")
        return cls(stochastic_duration=g("use_stochastic_duration_prediction", True),
                   duration_flows=g("duration_predictor_num_flows", 4), duration_flow_bins=g("duration_predictor_flow_bins", 10),
                   duration_tail_bound=g("duration_predictor_tail_bound", 5.0),
                   duration_stack_layers=g("depth_separable_num_layers", 3),
                   duration_dropout=g("duration_predictor_dropout", 0.5), noise_scale_duration=g("noise_scale_duration", 0.8),
                   vocab_size=g("vocab_size", 38), hidden=g("hidden_size", 192), layers=g("num_hidden_layers", 6),
                   heads=g("num_attention_heads", 2), window=g("window_size", 4), ffn=g("ffn_dim", 768),
                   ffn_kernel=g("ffn_kernel_size", 3), flow_size=g("flow_size", 192),
                   spectrogram_bins=g("spectrogram_bins", 513),
                   duration_filter=g("duration_predictor_filter_channels", 256),
                   duration_kernel=g("duration_predictor_kernel_size", 3), prior_flows=g("prior_encoder_num_flows", 4),
                   prior_wavenet_layers=g("prior_encoder_num_wavenet_layers", 4),
                   posterior_wavenet_layers=g("posterior_encoder_num_wavenet_layers", 16),
                   wavenet_kernel=g("wavenet_kernel_size", 5), wavenet_dilation=g("wavenet_dilation_rate", 1),
                   upsample_rates=tuple(g("upsample_rates", (8, 8, 2, 2))),
                   upsample_kernels=tuple(g("upsample_kernel_sizes", (16, 16, 4, 4))),
                   upsample_channels=g("upsample_initial_channel", 512),
                   resblock_kernels=tuple(g("resblock_kernel_sizes", (3, 7, 11))),
                   resblock_dilations=tuple(tuple(d) for d in g("resblock_dilation_sizes", ((1, 3, 5),) * 3)),
                   leaky_slope=g("leaky_relu_slope", 0.1), speakers=g("num_speakers", 1),
                   speaker_dim=g("speaker_embedding_size", 0), eps=g("layer_norm_eps", 1e-5),
                   noise_scale=g("noise_scale", 0.667), speaking_rate=g("speaking_rate", 1.0),
                   sampling_rate=g("sampling_rate", 16000), bias=g("use_bias", True))


def _randn(like: torch.Tensor, generator: Optional[torch.Generator], shape=None, uniform: bool = False) -> torch.Tensor:
    """Noise of ``like``'s shape (or ``shape``), dtype and device; drawn on the generator's own device when it has one."""
    shape = tuple(like.shape if shape is None else shape)
    device = like.device if generator is None else generator.device
    draw = torch.rand if uniform else torch.randn
    return draw(shape, device=device, dtype=torch.float32, generator=generator).to(device=like.device, dtype=like.dtype)


def length_mask(lengths: torch.Tensor, size: Optional[int] = None) -> torch.Tensor:
    """``[B, 1, T]`` float mask of the first ``lengths[b]`` positions."""
    size = int(lengths.max()) if size is None else size
    return (torch.arange(size, device=lengths.device)[None, :] < lengths[:, None]).unsqueeze(1).float()


# ------------------------------------------------------------------------------------------------------- text encoder
class WindowedRelativeAttention(nn.Module):
    """Self-attention whose logits and outputs get learned vectors for key offsets of at most ``window`` positions."""

    def __init__(self, s: VitsSpec):
        super().__init__()
        self.heads, self.dim, self.window = s.heads, s.hidden // s.heads, s.window
        self.q_proj = nn.Linear(s.hidden, s.hidden, bias=s.bias)
        self.k_proj = nn.Linear(s.hidden, s.hidden, bias=s.bias)
        self.v_proj = nn.Linear(s.hidden, s.hidden, bias=s.bias)
        self.out_proj = nn.Linear(s.hidden, s.hidden, bias=s.bias)
        if self.window:
            scale = self.dim ** -0.5
            self.emb_rel_k = nn.Parameter(torch.randn(1, 2 * s.window + 1, self.dim) * scale)
            self.emb_rel_v = nn.Parameter(torch.randn(1, 2 * s.window + 1, self.dim) * scale)

    def _offsets(self, T: int, device) -> torch.Tensor:
        """``[T, T]`` index of the offset ``j - i`` into the table, ``2 window + 1`` (a zero entry) outside the window."""
        d = torch.arange(T, device=device)[None, :] - torch.arange(T, device=device)[:, None]
        return torch.where(d.abs() <= self.window, d + self.window, torch.full_like(d, 2 * self.window + 1))

    def forward(self, x: torch.Tensor, key_mask: Optional[torch.Tensor]) -> torch.Tensor:
        """``x`` [B, T, C]; ``key_mask`` [B, T] (1 = a real token)."""
        B, T, _ = x.shape
        split = lambda t: t.view(B, T, self.heads, self.dim).transpose(1, 2)          # [B, H, T, D]
        q = split(self.q_proj(x)) * self.dim ** -0.5
        k, v = split(self.k_proj(x)), split(self.v_proj(x))
        logits = q @ k.transpose(-1, -2)
        if self.window:
            idx = self._offsets(T, x.device)
            rel = q @ self.emb_rel_k[0].t()                                          # [B, H, T, 2w+1]
            rel = F.pad(rel, (0, 1))                                                 # the zero entry
            logits = logits + rel.gather(-1, idx.expand(B, self.heads, T, T))
        if key_mask is not None:
            logits = logits.masked_fill(key_mask[:, None, None, :] == 0, torch.finfo(logits.dtype).min)
        p = logits.softmax(-1)
        out = p @ v
        if self.window:
            # weight of each offset: p[i, i + r - w]; outside the sequence it is zero
            r = torch.arange(2 * self.window + 1, device=x.device)[None, :]
            j = torch.arange(T, device=x.device)[:, None] + r - self.window          # [T, 2w+1]
            ok = (j >= 0) & (j < T)
            pr = p.gather(-1, j.clamp(0, T - 1).expand(B, self.heads, T, -1)) * ok
            out = out + pr @ self.emb_rel_v[0]
        return self.out_proj(out.transpose(1, 2).reshape(B, T, -1))


class ConvFeedForward(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        self.conv_1 = Conv1d(s.hidden, s.ffn, s.ffn_kernel)
        self.conv_2 = Conv1d(s.ffn, s.hidden, s.ffn_kernel)
        self.pad = ((s.ffn_kernel - 1) // 2, s.ffn_kernel // 2)

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """``x`` [B, C, T]; ``mask`` [B, 1, T]."""
        x = self.conv_1(F.pad(x * mask, self.pad))
        x = self.conv_2(F.pad(torch.relu(x) * mask, self.pad))
        return x * mask


class EncoderLayer(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        self.attention = WindowedRelativeAttention(s)
        self.layer_norm = nn.LayerNorm(s.hidden, eps=s.eps)
        self.feed_forward = ConvFeedForward(s)
        self.final_layer_norm = nn.LayerNorm(s.hidden, eps=s.eps)

    def forward(self, x, mask, key_mask):
        x = self.layer_norm(x + self.attention(x, key_mask))
        y = self.feed_forward(x.transpose(1, 2), mask).transpose(1, 2)
        return self.final_layer_norm(x + y)


class TextEncoder(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        self.spec = s
        self.embed_tokens = nn.Embedding(s.vocab_size, s.hidden)
        self.layers = nn.ModuleList(EncoderLayer(s) for _ in range(s.layers))
        self.project = Conv1d(s.hidden, 2 * s.flow_size, 1)

    def forward(self, ids: torch.Tensor, mask: torch.Tensor):
        """``ids`` [B, T]; ``mask`` [B, 1, T] -> hidden [B, C, T], prior mean and log-deviation [B, flow, T]."""
        key_mask = mask[:, 0]
        tm = mask.transpose(1, 2)
        x = self.embed_tokens(ids) * math.sqrt(self.spec.hidden) * tm
        for layer in self.layers:
            x = layer(x, mask, key_mask)
        x = (x * tm).transpose(1, 2)
        mean, log_dev = (self.project(x) * mask).split(self.spec.flow_size, dim=1)
        return x, mean, log_dev


# ------------------------------------------------------------------------------------------ wavenet, posterior, flow
class WaveNet(nn.Module):
    def __init__(self, s: VitsSpec, layers: int):
        super().__init__()
        self.hidden, self.n = s.hidden, layers
        self.in_layers = nn.ModuleList()
        self.res_skip_layers = nn.ModuleList()
        if s.speaker_dim:
            self.cond_layer = Conv1d(s.speaker_dim, 2 * s.hidden * layers, 1)
        for i in range(layers):
            d = s.wavenet_dilation ** i
            self.in_layers.append(Conv1d(s.hidden, 2 * s.hidden, s.wavenet_kernel, dilation=d,
                                         padding=(s.wavenet_kernel * d - d) // 2))
            self.res_skip_layers.append(Conv1d(s.hidden, 2 * s.hidden if i < layers - 1 else s.hidden, 1))

    def forward(self, x: torch.Tensor, mask: torch.Tensor, g: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.zeros_like(x)
        cond = self.cond_layer(g) if g is not None else None
        H = self.hidden
        for i in range(self.n):
            a = self.in_layers[i](x)
            if cond is not None:
                a = a + cond[:, 2 * H * i:2 * H * (i + 1)]
            a = torch.tanh(a[:, :H]) * torch.sigmoid(a[:, H:])
            rs = self.res_skip_layers[i](a)
            if i < self.n - 1:
                x = (x + rs[:, :H]) * mask
                out = out + rs[:, H:]
            else:
                out = out + rs
        return out * mask


class PosteriorEncoder(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        self.size = s.flow_size
        self.conv_pre = Conv1d(s.spectrogram_bins, s.hidden, 1)
        self.wavenet = WaveNet(s, s.posterior_wavenet_layers)
        self.conv_proj = Conv1d(s.hidden, 2 * s.flow_size, 1)

    def forward(self, spec, mask, g=None, generator: Optional[torch.Generator] = None):
        h = self.wavenet(self.conv_pre(spec) * mask, mask, g)
        mean, log_dev = (self.conv_proj(h) * mask).split(self.size, dim=1)
        noise = _randn(mean, generator)
        return (mean + noise * log_dev.exp()) * mask, mean, log_dev


class Coupling(nn.Module):
    """Mean-only coupling: the second half of the channels is shifted by a WaveNet of the first (volume preserving)."""

    def __init__(self, s: VitsSpec):
        super().__init__()
        self.half = s.flow_size // 2
        self.conv_pre = Conv1d(self.half, s.hidden, 1)
        self.wavenet = WaveNet(s, s.prior_wavenet_layers)
        self.conv_post = Conv1d(s.hidden, self.half, 1)

    def forward(self, x, mask, g=None, reverse: bool = False):
        a, b = x.split(self.half, dim=1)
        shift = self.conv_post(self.wavenet(self.conv_pre(a) * mask, mask, g)) * mask
        b = (b - shift) * mask if reverse else shift + b * mask
        return torch.cat([a, b], dim=1)


class Flow(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        self.flows = nn.ModuleList(Coupling(s) for _ in range(s.prior_flows))

    def forward(self, x, mask, g=None, reverse: bool = False):
        if not reverse:
            for f in self.flows:
                x = f(x, mask, g).flip(1)
        else:
            for f in reversed(self.flows):
                x = f(x.flip(1), mask, g, reverse=True)
        return x


class DurationPredictor(nn.Module):
    def __init__(self, s: VitsSpec):
        super().__init__()
        k = s.duration_kernel
        self.conv_1 = Conv1d(s.hidden, s.duration_filter, k, padding=k // 2)
        self.norm_1 = nn.LayerNorm(s.duration_filter, eps=s.eps)
        self.conv_2 = Conv1d(s.duration_filter, s.duration_filter, k, padding=k // 2)
        self.norm_2 = nn.LayerNorm(s.duration_filter, eps=s.eps)
        self.proj = Conv1d(s.duration_filter, 1, 1)
        if s.speaker_dim:
            self.cond = Conv1d(s.speaker_dim, s.hidden, 1)

    def forward(self, x, mask, g=None):
        """Log-frames per token ``[B, 1, T]``; the text encoder gets no gradient from here."""
        x = x.detach()
        if g is not None:
            x = x + self.cond(g.detach())
        x = self.norm_1(torch.relu(self.conv_1(x * mask)).transpose(1, 2)).transpose(1, 2)
        x = self.norm_2(torch.relu(self.conv_2(x * mask)).transpose(1, 2)).transpose(1, 2)
        return self.proj(x * mask) * mask



# ------------------------------------------------------------------------------------- stochastic duration predictor
def rational_quadratic_spline(x: torch.Tensor, width_logits: torch.Tensor, height_logits: torch.Tensor,
                              slope_logits: torch.Tensor, inverse: bool = False, bound: float = 5.0,
                              min_width: float = 1e-3, min_height: float = 1e-3, min_slope: float = 1e-3):
    """Monotone piecewise rational-quadratic map of ``[-bound, bound]`` onto itself (Durkan et al., neural spline
    flows), the identity outside. ``width_logits`` / ``height_logits`` ``[..., K]`` give the K bins, ``slope_logits``
    ``[..., K - 1]`` the derivatives at the inner knots (1 at both ends). Returns the mapped values and the log of the
    derivative of the forward map at them (of the inverse map's input when ``inverse``: negate for its own)."""
    K = width_logits.shape[-1]
    inside = (x >= -bound) & (x <= bound)
    xc = x.clamp(-bound, bound)

    def knots(logits, floor):
        sizes = floor + (1 - floor * K) * logits.softmax(-1)
        edges = F.pad(sizes.cumsum(-1), (1, 0)) * 2 * bound - bound
        edges = torch.cat([edges[..., :1] * 0 - bound, edges[..., 1:-1], edges[..., -1:] * 0 + bound], -1)
        return edges, edges[..., 1:] - edges[..., :-1]

    xk, w = knots(width_logits, min_width)
    yk, h = knots(height_logits, min_height)
    end = math.log(math.exp(1 - min_slope) - 1)                                   # softplus^-1(1 - min_slope)
    d = min_slope + F.softplus(F.pad(slope_logits, (1, 1), value=end))
    search = (yk if inverse else xk).clone()
    search[..., -1] += 1e-6
    k = ((xc[..., None] >= search).sum(-1) - 1).clamp(0, K - 1)[..., None]
    pick = lambda t: t.gather(-1, k)[..., 0]
    x0, w0, y0, h0 = pick(xk), pick(w), pick(yk), pick(h)
    s = h0 / w0
    d0, d1 = pick(d), pick(d[..., 1:])
    bend = d0 + d1 - 2 * s
    if not inverse:
        t = (xc - x0) / w0
        tt = t * (1 - t)
        den = s + bend * tt
        y = y0 + h0 * (s * t * t + d0 * tt) / den
        logdet = torch.log(s * s * (d1 * t * t + 2 * s * tt + d0 * (1 - t) ** 2)) - 2 * torch.log(den)
    else:
        dy = xc - y0
        a = h0 * (s - d0) + dy * bend
        b = h0 * d0 - dy * bend
        c = -s * dy
        t = 2 * c / (-b - torch.sqrt((b * b - 4 * a * c).clamp_min(0)))
        tt = t * (1 - t)
        den = s + bend * tt
        y = t * w0 + x0
        logdet = torch.log(s * s * (d1 * t * t + 2 * s * tt + d0 * (1 - t) ** 2)) - 2 * torch.log(den)
    return torch.where(inside, y, x), torch.where(inside, logdet, torch.zeros_like(logdet))


class SeparableConvStack(nn.Module):
    """Residual layers of a dilated depthwise convolution and a pointwise one, each followed by LayerNorm + GELU."""

    def __init__(self, s: VitsSpec, dropout: float = 0.0):
        super().__init__()
        k, c = s.duration_kernel, s.hidden
        self.convs_dilated = nn.ModuleList(Conv1d(c, c, k, groups=c, dilation=k ** i, padding=(k * k ** i - k ** i) // 2)
                                           for i in range(s.duration_stack_layers))
        self.convs_pointwise = nn.ModuleList(Conv1d(c, c, 1) for _ in range(s.duration_stack_layers))
        self.norms_1 = nn.ModuleList(nn.LayerNorm(c) for _ in range(s.duration_stack_layers))
        self.norms_2 = nn.ModuleList(nn.LayerNorm(c) for _ in range(s.duration_stack_layers))
        self.dropout = nn.Dropout(dropout)

    def forward(self, x, mask, g=None):
        if g is not None:
            x = x + g
        for dw, pw, n1, n2 in zip(self.convs_dilated, self.convs_pointwise, self.norms_1, self.norms_2):
            h = F.gelu(n1(dw(x * mask).transpose(1, 2)).transpose(1, 2))
            h = F.gelu(n2(pw(h).transpose(1, 2)).transpose(1, 2))
            x = x + self.dropout(h)
        return x * mask


class SplineCoupling(nn.Module):
    """Two channels: the second goes through a spline whose bins come from the first (and the condition)."""

    def __init__(self, s: VitsSpec):
        super().__init__()
        self.bins, self.bound, self.scale = s.duration_flow_bins, s.duration_tail_bound, math.sqrt(s.hidden)
        self.conv_pre = Conv1d(1, s.hidden, 1)
        self.conv_dds = SeparableConvStack(s)
        self.conv_proj = Conv1d(s.hidden, 3 * s.duration_flow_bins - 1, 1)

    def forward(self, x, mask, g=None, reverse: bool = False):
        a, b = x.split(1, dim=1)
        h = self.conv_proj(self.conv_dds(self.conv_pre(a), mask, g)) * mask        # [B, 3K-1, T]
        h = h.transpose(1, 2).unsqueeze(1)                                         # [B, 1, T, 3K-1]
        K = self.bins
        b, logdet = rational_quadratic_spline(b, h[..., :K] / self.scale, h[..., K:2 * K] / self.scale, h[..., 2 * K:],
                                              inverse=reverse, bound=self.bound)
        return torch.cat([a, b], dim=1) * mask, (logdet * mask).sum((1, 2))


class ChannelAffine(nn.Module):
    def __init__(self, channels: int = 2):
        super().__init__()
        self.translate = nn.Parameter(torch.zeros(channels, 1))
        self.log_scale = nn.Parameter(torch.zeros(channels, 1))

    def forward(self, x, mask, g=None, reverse: bool = False):
        if reverse:
            return (x - self.translate) * torch.exp(-self.log_scale) * mask, None
        return (self.translate + torch.exp(self.log_scale) * x) * mask, (self.log_scale * mask).sum((1, 2))


class StochasticDurationPredictor(nn.Module):
    """A flow over (log-duration, companion) pairs per token, conditioned on the text: sampled backwards for synthesis,
    trained forwards by a variational bound in which a second flow de-quantises the integer durations."""

    def __init__(self, s: VitsSpec):
        super().__init__()
        c = s.hidden
        self.conv_pre, self.conv_proj = Conv1d(c, c, 1), Conv1d(c, c, 1)
        self.conv_dds = SeparableConvStack(s, s.duration_dropout)
        if s.speaker_dim:
            self.cond = Conv1d(s.speaker_dim, c, 1)
        self.flows = nn.ModuleList([ChannelAffine()] + [SplineCoupling(s) for _ in range(s.duration_flows)])
        self.post_conv_pre, self.post_conv_proj = Conv1d(1, c, 1), Conv1d(c, c, 1)
        self.post_conv_dds = SeparableConvStack(s, s.duration_dropout)
        self.post_flows = nn.ModuleList([ChannelAffine()] + [SplineCoupling(s) for _ in range(s.duration_flows)])

    def _condition(self, x, mask, g):
        x = self.conv_pre(x.detach())
        if g is not None:
            x = x + self.cond(g.detach())
        return self.conv_proj(self.conv_dds(x, mask)) * mask

    def forward(self, x, mask, g=None, noise_scale: float = 1.0, generator: Optional[torch.Generator] = None):
        """Sampled log-frames per token ``[B, 1, T]``."""
        cond = self._condition(x, mask, g)
        z = _randn(x, generator, (x.shape[0], 2, x.shape[2])) * noise_scale
        order = list(reversed(self.flows))
        order = order[:-2] + [order[-1]]                   # the published sampler skips the coupling next to the affine map
        for f in order:
            z, _ = f(z.flip(1), mask, cond, reverse=True)
        return z[:, :1]

    def negative_log_likelihood(self, x, mask, durations, g=None, generator: Optional[torch.Generator] = None):
        """Variational upper bound of -log p(durations | text) per sequence ``[B]``; ``durations`` [B, 1, T] frames."""
        cond = self._condition(x, mask, g)
        post = self.post_conv_proj(self.post_conv_dds(self.post_conv_pre(durations), mask)) * mask
        e = _randn(x, generator, (x.shape[0], 2, x.shape[2])) * mask
        z, logdet_q = e, 0.0
        for f in self.post_flows:
            z, ld = f(z, mask, cond + post)
            z, logdet_q = z.flip(1), logdet_q + ld
        u, v = z.split(1, dim=1)
        logdet_q = logdet_q + ((F.logsigmoid(u) + F.logsigmoid(-u)) * mask).sum((1, 2))
        log_q = (-0.5 * (math.log(2 * math.pi) + e * e) * mask).sum((1, 2)) - logdet_q
        first = torch.log(((durations - torch.sigmoid(u)) * mask).clamp_min(1e-5)) * mask
        logdet = (-first).sum((1, 2))
        z = torch.cat([first, v], dim=1)
        for f in self.flows:
            z, ld = f(z, mask, cond)
            z, logdet = z.flip(1), logdet + ld
        nll = (0.5 * (math.log(2 * math.pi) + z * z) * mask).sum((1, 2)) - logdet
        return nll + log_q


# --------------------------------------------------------------------------------------------------------- generator
class ResidualBlock(nn.Module):
    def __init__(self, channels: int, kernel: int, dilations: Sequence[int], slope: float):
        super().__init__()
        self.slope = slope
        self.convs1 = nn.ModuleList(Conv1d(channels, channels, kernel, dilation=d, padding=(kernel * d - d) // 2)
                                    for d in dilations)
        self.convs2 = nn.ModuleList(Conv1d(channels, channels, kernel, padding=(kernel - 1) // 2) for _ in dilations)

    def forward(self, x):
        for c1, c2 in zip(self.convs1, self.convs2):
            x = x + c2(F.leaky_relu(c1(F.leaky_relu(x, self.slope)), self.slope))
        return x


class Generator(nn.Module):
    """HiFi-GAN: latent frames ``[B, flow, T]`` -> waveform ``[B, 1, T x hop]``."""

    def __init__(self, s: VitsSpec):
        super().__init__()
        self.slope, self.kernels = s.leaky_slope, len(s.resblock_kernels)
        self.conv_pre = Conv1d(s.flow_size, s.upsample_channels, 7, padding=3)
        self.upsampler = nn.ModuleList()
        self.resblocks = nn.ModuleList()
        ch = s.upsample_channels
        for rate, k in zip(s.upsample_rates, s.upsample_kernels):
            self.upsampler.append(nn.ConvTranspose1d(ch, ch // 2, k, stride=rate, padding=(k - rate) // 2))
            ch //= 2
            for rk, rd in zip(s.resblock_kernels, s.resblock_dilations):
                self.resblocks.append(ResidualBlock(ch, rk, rd, s.leaky_slope))
        self.conv_post = Conv1d(ch, 1, 7, padding=3, bias=False)
        if s.speaker_dim:
            self.cond = Conv1d(s.speaker_dim, s.upsample_channels, 1)

    def forward(self, z, g=None):
        x = self.conv_pre(z)
        if g is not None:
            x = x + self.cond(g)
        for i, up in enumerate(self.upsampler):
            x = up(F.leaky_relu(x, self.slope))
            blocks = self.resblocks[i * self.kernels:(i + 1) * self.kernels]
            x = sum(b(x) for b in blocks) / self.kernels
        return torch.tanh(self.conv_post(F.leaky_relu(x)))               # the last slope is the default 0.01


# --------------------------------------------------------------------------------------------------------- alignment
def monotonic_alignment(score: torch.Tensor, frames: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """The 0 / 1 alignment ``[B, F, T]`` that maximises the summed ``score[b, f, t]`` over paths in which frame 0 maps
    to token 0, the last frame to the last token, and the token index never decreases nor skips (so every token gets at
    least one frame; ``frames[b] >= tokens[b]`` is required). Dynamic programme over the frames, all sequences and
    tokens at once; the backward walk is batched too."""
    B, Fm, Tm = score.shape
    if bool((frames < tokens).any()):
        raise ValueError("monotonic alignment needs at least one frame per token")
    if score.is_cuda:
        return _monotonic_alignment_device(score, frames, tokens)
    neg = torch.finfo(score.dtype).min / 4
    tok = torch.arange(Tm, device=score.device)[None, :]
    value = torch.full((B, Fm, Tm), neg, dtype=score.dtype, device=score.device)
    prev = torch.full((B, Tm), neg, dtype=score.dtype, device=score.device)
    for f in range(Fm):
        if f == 0:
            cur = torch.where(tok == 0, score[:, 0], torch.full_like(prev, neg))
        else:
            diag = torch.cat([torch.full_like(prev[:, :1], neg), prev[:, :-1]], dim=1)
            cur = score[:, f] + torch.maximum(prev, diag)
            cur = torch.where(tok <= f, cur, torch.full_like(cur, neg))
        cur = cur.clamp_min(neg)
        value[:, f] = cur
        prev = cur
    path = torch.zeros_like(score)
    rows = torch.arange(B, device=score.device)
    idx = (tokens - 1).clone()
    for f in range(Fm - 1, -1, -1):
        active = f < frames
        path[rows[active], f, idx[active]] = 1.0
        if f == 0:
            break
        stay = value[rows, f - 1, idx]
        step = value[rows, f - 1, (idx - 1).clamp_min(0)]
        move = active & (f < frames) & (idx > 0) & ((idx == f) | (stay < step))
        # the first active row of a sequence is its last frame: it keeps the last token
        idx = idx - move.long()
    return path


def _monotonic_alignment_device(score: torch.Tensor, frames: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """The same search as one launch (``csrc/align.cu``): one CTA per sequence, rows of best totals in shared memory."""
    from .. import _native
    from ..ops._util import stream_ptr
    B, Fm, Tm = score.shape
    sc = score.float().contiguous()
    fr, tk = frames.to(torch.int32).contiguous(), tokens.to(torch.int32).contiguous()
    path = torch.zeros_like(sc)
    step = torch.empty((B, Fm, Tm), dtype=torch.uint8, device=sc.device)
    rows = torch.empty((B, 2, Tm) if Tm > 6000 else (1,), dtype=torch.float32, device=sc.device)
    rc = _native.lib().idrak_monotonic_align(sc.data_ptr(), fr.data_ptr(), tk.data_ptr(), path.data_ptr(), step.data_ptr(),
                                             rows.data_ptr(), B, Fm, Tm, stream_ptr())
    _native.check(rc, "idrak_monotonic_align")
    return path.to(score.dtype)


def prior_scores(z: torch.Tensor, mean: torch.Tensor, log_dev: torch.Tensor) -> torch.Tensor:
    """``[B, F, T]`` log-density of every latent frame ``z[:, :, f]`` under every token's Gaussian prior."""
    inv_var = torch.exp(-2 * log_dev)                                                 # [B, C, T]
    const = (-0.5 * math.log(2 * math.pi) - log_dev).sum(1, keepdim=True)             # [B, 1, T]
    quad = (-0.5 * z * z).transpose(1, 2) @ inv_var                                   # [B, F, T]
    cross = z.transpose(1, 2) @ (mean * inv_var)
    mean_sq = (-0.5 * mean * mean * inv_var).sum(1, keepdim=True)
    return const + quad + cross + mean_sq


def expand_by_durations(values: torch.Tensor, durations: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Repeat each token's column ``durations[b, t]`` times: ``values`` [B, C, T] -> ([B, C, F], frame counts [B])."""
    cum = durations.long().cumsum(-1)                                                 # [B, T]
    total = cum[:, -1].clamp_min(1)
    Fm = int(total.max())
    frame = torch.arange(Fm, device=values.device)[None, :].expand(values.shape[0], -1).contiguous()
    token = torch.searchsorted(cum, frame, right=True).clamp_max(values.shape[-1] - 1)
    out = values.gather(2, token[:, None, :].expand(-1, values.shape[1], -1))
    return out * length_mask(total, Fm).to(values.dtype), total


# -------------------------------------------------------------------------------------------------------------- model
class Vits(nn.Module):
    def __init__(self, spec: VitsSpec):
        super().__init__()
        self.spec = spec
        self.text_encoder = TextEncoder(spec)
        self.flow = Flow(spec)
        self.decoder = Generator(spec)
        self.duration_predictor = StochasticDurationPredictor(spec) if spec.stochastic_duration else DurationPredictor(spec)
        self.posterior_encoder = PosteriorEncoder(spec)
        if spec.speakers > 1:
            self.embed_speaker = nn.Embedding(spec.speakers, spec.speaker_dim)

    @property
    def dtype(self) -> torch.dtype:
        return self.text_encoder.embed_tokens.weight.dtype

    def _speaker(self, speaker: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if speaker is None or self.spec.speakers <= 1:
            return None
        return self.embed_speaker(speaker).unsqueeze(-1)

    @torch.no_grad()
    def synthesize(self, ids: torch.Tensor, lengths: Optional[torch.Tensor] = None, speaker: Optional[torch.Tensor] = None,
                   noise_scale: Optional[float] = None, speaking_rate: Optional[float] = None,
                   generator: Optional[torch.Generator] = None,
                   noise_scale_duration: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Token ids ``[B, T]`` -> (waveform ``[B, samples]``, valid samples per sequence ``[B]``)."""
        s = self.spec
        lengths = torch.full((ids.shape[0],), ids.shape[1], device=ids.device) if lengths is None else lengths
        mask = length_mask(lengths, ids.shape[1]).to(self.dtype)
        g = self._speaker(speaker)
        hidden, mean, log_dev = self.text_encoder(ids, mask)
        if s.stochastic_duration:
            nsd = s.noise_scale_duration if noise_scale_duration is None else noise_scale_duration
            log_frames = self.duration_predictor(hidden, mask, g, nsd, generator)
        else:
            log_frames = self.duration_predictor(hidden, mask, g)
        rate = s.speaking_rate if speaking_rate is None else speaking_rate
        durations = torch.ceil(log_frames.exp() * mask / rate)[:, 0]
        mean, frames = expand_by_durations(mean, durations)
        log_dev, _ = expand_by_durations(log_dev, durations)
        out_mask = length_mask(frames, mean.shape[-1]).to(self.dtype)
        scale = s.noise_scale if noise_scale is None else noise_scale
        noise = _randn(mean, generator)
        z = self.flow(mean + noise * log_dev.exp() * scale, out_mask, g, reverse=True) * out_mask
        return self.decoder(z, g)[:, 0], frames * s.hop

    @torch.no_grad()
    def convert_voice(self, spectrogram: torch.Tensor, lengths: torch.Tensor, source: torch.Tensor, target: torch.Tensor,
                      tau: float = 0.0, generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Re-voice a recording: its spectrogram ``[B, bins, F]`` is encoded under the ``source`` speaker, carried
        through the flow into the speaker-free prior space and back under the ``target`` speaker, then generated.
        ``source`` / ``target`` are speaker ids ``[B]`` or embeddings ``[B, speaker_dim, 1]`` (for instance from a
        ``ReferenceEncoder``); ``tau`` scales the posterior's sampling noise (0 = its mean)."""
        as_g = lambda v: v if v.dim() == 3 else self.embed_speaker(v).unsqueeze(-1)
        g_src, g_tgt = as_g(source), as_g(target)
        mask = length_mask(lengths, spectrogram.shape[-1]).to(self.dtype)
        z, mean, _ = self.posterior_encoder(spectrogram, mask, g_src, generator)
        z = mean + (z - mean) * tau
        z = self.flow(self.flow(z, mask, g_src), mask, g_tgt, reverse=True) * mask
        return self.decoder(z, g_tgt)[:, 0], lengths * self.spec.hop

    def training_losses(self, ids: torch.Tensor, id_lengths: torch.Tensor, spectrogram: torch.Tensor,
                        spec_lengths: torch.Tensor, speaker: Optional[torch.Tensor] = None, segment: int = 32,
                        generator: Optional[torch.Generator] = None) -> Dict[str, torch.Tensor]:
        """One generator-side pass: ``duration`` and ``kl`` losses, the generated waveform ``segment_wave``
        ``[B, 1, segment x hop]`` of a random window of latent frames and that window's first frame ``segment_start``
        (to cut the same samples from the recording for the spectral and adversarial losses), and the alignment."""
        mask = length_mask(id_lengths, ids.shape[1]).to(self.dtype)
        smask = length_mask(spec_lengths, spectrogram.shape[-1]).to(self.dtype)
        g = self._speaker(speaker)
        hidden, mean_p, log_dev_p = self.text_encoder(ids, mask)
        z, mean_q, log_dev_q = self.posterior_encoder(spectrogram, smask, g, generator)
        z_p = self.flow(z, smask, g)
        with torch.no_grad():
            align = monotonic_alignment(prior_scores(z_p, mean_p, log_dev_p), spec_lengths, id_lengths)
        frames_per_token = align.sum(1)                                               # [B, T]
        if self.spec.stochastic_duration:
            nll = self.duration_predictor.negative_log_likelihood(hidden, mask, frames_per_token.unsqueeze(1), g, generator)
            duration = (nll / mask.sum((1, 2))).sum()
        else:
            target = torch.log(frames_per_token + 1e-6).unsqueeze(1) * mask
            log_frames = self.duration_predictor(hidden, mask, g)
            duration = ((log_frames - target) ** 2 * mask).sum() / mask.sum()
        mean_f = mean_p @ align.transpose(1, 2)                                       # [B, C, F]
        log_dev_f = log_dev_p @ align.transpose(1, 2)
        kl = log_dev_f - log_dev_q - 0.5 + 0.5 * (z_p - mean_f) ** 2 * torch.exp(-2 * log_dev_f)
        kl = (kl * smask).sum() / smask.sum()
        seg = min(segment, int(spec_lengths.min()))
        high = (spec_lengths - seg + 1).clamp_min(1).float()
        u = _randn(high, generator, uniform=True)
        start = (u * high).long()
        cols = start[:, None] + torch.arange(seg, device=z.device)[None, :]
        z_seg = z.gather(2, cols[:, None, :].expand(-1, z.shape[1], -1))
        return {"duration": duration, "kl": kl, "segment_wave": self.decoder(z_seg, g), "segment_start": start,
                "segment_frames": torch.tensor(seg), "alignment": align}

    # ---------------------------------------------------------------------------------------------------- loading
    def load_hf_state(self, state: Dict[str, torch.Tensor]) -> None:
        """Load a Hugging Face ``VitsModel`` state dict (weight-normalised convolutions folded into plain weights)."""
        plain: Dict[str, torch.Tensor] = {}
        for name, t in state.items():
            if name.endswith("parametrizations.weight.original0"):
                base = name[:-len("parametrizations.weight.original0")]
                gain, direction = t.float(), state[base + "parametrizations.weight.original1"].float()
                norm = direction.flatten(1).norm(dim=1).view(-1, *[1] * (direction.dim() - 1))
                plain[base + "weight"] = (gain * direction / norm).to(t.dtype)
            elif name.endswith("parametrizations.weight.original1"):
                continue
            elif name.endswith("weight_g"):                                     # the older weight-norm spelling
                direction = state[name[:-2] + "_v"].float()
                norm = direction.flatten(1).norm(dim=1).view(-1, *[1] * (direction.dim() - 1))
                plain[name[:-2]] = (t.float() * direction / norm).to(t.dtype)
            elif name.endswith("weight_v"):
                continue
            else:
                plain[name.replace("text_encoder.encoder.layers.", "text_encoder.layers.")] = t
        missing, unexpected = self.load_state_dict(plain, strict=False)
        if missing or unexpected:
            raise KeyError(f"VITS state mismatch: missing {list(missing)[:5]}, unexpected {list(unexpected)[:5]}")


class ReferenceEncoder(nn.Module):
    """A speaker (tone colour) embedding ``[B, speaker_dim, 1]`` from a spectrogram of any length: strided 2-D
    convolutions over (frequency, time), a GRU over the remaining frames, a projection of its last state."""

    def __init__(self, bins: int, speaker_dim: int, channels: Sequence[int] = (32, 32, 64, 64, 128, 128), hidden: int = 128):
        super().__init__()
        layers, prev = [], 1
        for c in channels:
            layers += [nn.Conv2d(prev, c, 3, 2, 1), nn.ReLU()]
            prev = c
            bins = (bins - 1) // 2 + 1
        self.convs = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(bins * prev)
        self.gru = nn.GRU(bins * prev, hidden, batch_first=True)
        self.proj = nn.Linear(hidden, speaker_dim)

    def forward(self, spectrogram: torch.Tensor) -> torch.Tensor:
        x = self.convs(spectrogram.unsqueeze(1))                                  # [B, C, bins', F']
        x = x.permute(0, 3, 1, 2).flatten(2)                                      # [B, F', C x bins']
        _, h = self.gru(self.norm(x))
        return self.proj(h[-1]).unsqueeze(-1)


# ---------------------------------------------------------------------------------------------------- discriminators
class PeriodDiscriminator(nn.Module):
    """The waveform folded into ``[T / period, period]`` and convolved along the first axis only."""

    def __init__(self, period: int, channels: Sequence[int] = (32, 128, 512, 1024, 1024)):
        super().__init__()
        self.period = period
        layers, prev = [], 1
        for i, c in enumerate(channels):
            layers.append(nn.Conv2d(prev, c, (5, 1), (3 if i < len(channels) - 1 else 1, 1), padding=(2, 0)))
            prev = c
        self.convs = nn.ModuleList(layers)
        self.post = nn.Conv2d(prev, 1, (3, 1), padding=(1, 0))

    def forward(self, wave: torch.Tensor) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        B, C, T = wave.shape
        if T % self.period:
            wave = F.pad(wave, (0, self.period - T % self.period), mode="reflect")
        x = wave.view(B, C, -1, self.period)
        features = []
        for conv in self.convs:
            x = F.leaky_relu(conv(x), 0.1)
            features.append(x)
        x = self.post(x)
        features.append(x)
        return x.flatten(1), features


class ScaleDiscriminator(nn.Module):
    """Grouped strided 1-D convolutions over the raw waveform."""

    def __init__(self, width: int = 16):
        super().__init__()
        w = width
        self.convs = nn.ModuleList([
            nn.Conv1d(1, w, 15, 1, padding=7), nn.Conv1d(w, 4 * w, 41, 4, groups=4, padding=20),
            nn.Conv1d(4 * w, 16 * w, 41, 4, groups=16, padding=20), nn.Conv1d(16 * w, 64 * w, 41, 4, groups=64, padding=20),
            nn.Conv1d(64 * w, 64 * w, 41, 4, groups=256 if 64 * w % 256 == 0 else 64, padding=20),
            nn.Conv1d(64 * w, 64 * w, 5, 1, padding=2)])
        self.post = nn.Conv1d(64 * w, 1, 3, 1, padding=1)

    def forward(self, wave):
        x, features = wave, []
        for conv in self.convs:
            x = F.leaky_relu(conv(x), 0.1)
            features.append(x)
        x = self.post(x)
        features.append(x)
        return x.flatten(1), features


class Discriminators(nn.Module):
    def __init__(self, periods: Sequence[int] = (2, 3, 5, 7, 11), period_channels: Sequence[int] = (32, 128, 512, 1024, 1024),
                 scale_width: int = 16):
        super().__init__()
        self.branches = nn.ModuleList([ScaleDiscriminator(scale_width)] +
                                      [PeriodDiscriminator(p, period_channels) for p in periods])

    def forward(self, wave: torch.Tensor):
        """Per branch: (scores ``[B, n]``, feature maps)."""
        return [b(wave) for b in self.branches]


def discriminator_loss(real, fake) -> torch.Tensor:
    """Least squares: real scores towards 1, generated towards 0."""
    return sum(((1 - r[0]) ** 2).mean() + (f[0] ** 2).mean() for r, f in zip(real, fake))


def generator_adversarial_loss(fake) -> torch.Tensor:
    return sum(((1 - f[0]) ** 2).mean() for f in fake)


def feature_matching_loss(real, fake) -> torch.Tensor:
    return 2 * sum((a.detach() - b).abs().mean() for r, f in zip(real, fake) for a, b in zip(r[1], f[1]))


def linear_spectrogram(wave: torch.Tensor, n_fft: int = 1024, hop: int = 256, window: Optional[int] = None) -> torch.Tensor:
    """Magnitude spectrogram ``[B, n_fft / 2 + 1, frames]`` with reflect padding so that frames = samples / hop."""
    window = window or n_fft
    pad = (n_fft - hop) // 2
    x = F.pad(wave.unsqueeze(1), (pad, pad), mode="reflect").squeeze(1)
    spec = torch.stft(x, n_fft, hop_length=hop, win_length=window, window=torch.hann_window(window, device=wave.device),
                      center=False, return_complex=True)
    return torch.sqrt(spec.real ** 2 + spec.imag ** 2 + 1e-6)


def mel_from_linear(spec: torch.Tensor, sampling_rate: int, mels: int = 80) -> torch.Tensor:
    """Log-mel ``[B, mels, frames]`` of a magnitude spectrogram (this package's mel filter bank)."""
    from . import mel_filters
    n_fft = (spec.shape[1] - 1) * 2
    bank = torch.as_tensor(mel_filters(sampling_rate, n_fft, mels), dtype=spec.dtype, device=spec.device)
    return torch.log((bank @ spec).clamp_min(1e-5))


def slice_wave(wave: torch.Tensor, start_frames: torch.Tensor, frames: int, hop: int) -> torch.Tensor:
    """``[B, 1, frames x hop]`` windows of ``wave`` [B, samples] starting at ``start_frames x hop``."""
    cols = (start_frames * hop)[:, None] + torch.arange(frames * hop, device=wave.device)[None, :]
    return wave.gather(1, cols.clamp_max(wave.shape[1] - 1)).unsqueeze(1)


# ------------------------------------------------------------------------------------------------------------ trainer
class VitsTrainer:
    """Alternating discriminator / generator updates over (tokens, recording) batches.

    Without ``discriminators`` the generator trains on the spectral, KL and duration terms alone (plain TTS training);
    with them each step first updates the discriminators on the real and the detached generated window, then the
    generator with the adversarial and feature-matching terms added. The spectrogram of the recording is computed
    here (``n_fft`` must give ``spec.spectrogram_bins = n_fft / 2 + 1`` and the hop is the generator's up-sampling)."""

    def __init__(self, model: Vits, discriminators: Optional[Discriminators] = None, lr: float = 2e-4,
                 betas: Tuple[float, float] = (0.8, 0.99), spectral_weight: float = 45.0, kl_weight: float = 1.0,
                 segment: int = 32, mels: int = 0, seed: int = 0):
        self.model, self.disc = model, discriminators
        self.n_fft = (model.spec.spectrogram_bins - 1) * 2
        self.spectral_weight, self.kl_weight, self.segment, self.mels = spectral_weight, kl_weight, segment, mels
        self.opt_g = torch.optim.AdamW(model.parameters(), lr=lr, betas=betas, eps=1e-9)
        self.opt_d = None if discriminators is None else torch.optim.AdamW(discriminators.parameters(), lr=lr, betas=betas, eps=1e-9)
        self.generator = torch.Generator().manual_seed(seed)
        self.steps = 0

    def _spectral(self, wave: torch.Tensor) -> torch.Tensor:
        lin = linear_spectrogram(wave, self.n_fft, self.model.spec.hop)
        return mel_from_linear(lin, self.model.spec.sampling_rate, self.mels) if self.mels else lin.log()

    def step(self, ids: torch.Tensor, id_lengths: torch.Tensor, wave: torch.Tensor, wave_lengths: torch.Tensor,
             speaker: Optional[torch.Tensor] = None) -> Dict[str, float]:
        m, hop = self.model, self.model.spec.hop
        lin = linear_spectrogram(wave, self.n_fft, hop)
        frames = (wave_lengths // hop).clamp(1, lin.shape[-1])
        out = m.training_losses(ids, id_lengths, lin, frames, speaker, self.segment, self.generator)
        seg = int(out["segment_frames"])
        real = slice_wave(wave, out["segment_start"], seg, hop)
        report: Dict[str, float] = {}
        if self.disc is not None:
            d_loss = discriminator_loss(self.disc(real), self.disc(out["segment_wave"].detach()))
            self.opt_d.zero_grad(set_to_none=True)
            d_loss.backward()
            self.opt_d.step()
            report["discriminator"] = float(d_loss.detach())
        spectral = (self._spectral(out["segment_wave"][:, 0]) - self._spectral(real[:, 0])).abs().mean()
        loss = self.spectral_weight * spectral + self.kl_weight * out["kl"] + out["duration"]
        if self.disc is not None:
            fake_scores, real_scores = self.disc(out["segment_wave"]), self.disc(real)
            adv, fm = generator_adversarial_loss(fake_scores), feature_matching_loss(real_scores, fake_scores)
            loss = loss + adv + fm
            report.update(adversarial=float(adv.detach()), feature_matching=float(fm.detach()))
        self.opt_g.zero_grad(set_to_none=True)
        loss.backward()
        self.opt_g.step()
        self.steps += 1
        report.update(loss=float(loss.detach()), spectral=float(spectral.detach()), kl=float(out["kl"].detach()),
                      duration=float(out["duration"].detach()))
        return report
