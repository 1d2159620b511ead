"""General-purpose layers (beyond the decoder): dense, embedding, norms, attention, transformer encoder, recurrent,
convolution and pooling - and the layer-type registry that describes each as JSON and rebuilds it.

Dense, LayerNorm, RMSNorm, embedding and attention run on this package's kernels when their inputs are bf16 CUDA
tensors (``ops.linear`` -> the tcgen05 GEMM with fused bias / residual; ``ops.layer_norm``; flash attention); other
dtypes and the convolution / pooling / recurrent layers use the library's kernels.

Reference: src/Idrak/Layers (Linear.cs:13, Embedding.cs:13, Normalization.cs, Attention.cs:22,484,788, Recurrent.cs,
Convolution.cs, Sequential.cs:22) and the layer-type table of LibraryLayerTypes.cs:17-116 (type names and fields).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..core.registry import SlotTable
from ..ops import conv as conv_ops
from ..ops import reduce as ops_reduce
from ..ops import recurrent as recurrent_ops


def _fast(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if bias:
            bound = 1 / math.sqrt(in_features)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x, residual=None):
        if _fast(x) and self.in_features % 8 == 0 and self.out_features % 8 == 0:   # 16-byte rows on both sides
            return ops.linear(x, self.weight, self.bias, residual)
        y = F.linear(x, self.weight, self.bias)
        return y if residual is None else y + residual


class Embedding(nn.Module):
    def __init__(self, vocabulary: int, dim: int):
        super().__init__()
        self.vocabulary, self.dim = vocabulary, dim
        self.weight = nn.Parameter(torch.randn(vocabulary, dim) * 0.02)

    def forward(self, ids):
        return F.embedding(ids.long(), self.weight)


class LayerNorm(nn.Module):
    def __init__(self, features: int, epsilon: float = 1e-5):
        super().__init__()
        self.features, self.epsilon = features, epsilon
        self.weight, self.bias = nn.Parameter(torch.ones(features)), nn.Parameter(torch.zeros(features))

    def forward(self, x):
        if _fast(x) and self.features % 8 == 0:
            return ops.layer_norm(x, self.weight, self.bias, self.epsilon)
        return F.layer_norm(x, (self.features,), self.weight, self.bias, self.epsilon)


class RMSNorm(nn.Module):
    def __init__(self, features: int, epsilon: float = 1e-6):
        super().__init__()
        self.features, self.epsilon = features, epsilon
        self.weight = nn.Parameter(torch.ones(features))

    def forward(self, x):
        if _fast(x) and self.features % 8 == 0:
            return ops.rms_norm(x, self.weight, self.epsilon)
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.epsilon)).to(x.dtype) * self.weight


class PositionalEncoding(nn.Module):
    """Fixed sinusoids added to ``[N, T, dim]``."""

    def __init__(self, max_length: int, dim: int):
        super().__init__()
        self.max_length, self.dim = max_length, dim
        pos = torch.arange(max_length)[:, None].float()
        div = torch.exp(torch.arange(0, dim, 2).float() * (-math.log(10000.0) / dim))
        table = torch.zeros(max_length, dim)
        table[:, 0::2] = torch.sin(pos * div)
        table[:, 1::2] = torch.cos(pos * div)[:, : dim // 2]
        self.register_buffer("table", table, persistent=False)

    def forward(self, x):
        return x + self.table[: x.shape[1]].to(x.dtype)


class MultiHeadAttention(nn.Module):
    """Self-attention over ``[N, T, dim]`` (packed q/k/v projection), optionally causal; ``key_padding`` marks
    padded positions (True = ignore)."""

    def __init__(self, dim: int, heads: int, causal: bool = False, dropout: float = 0.0):
        super().__init__()
        if dim % heads:
            raise ValueError("dim must be a multiple of heads")
        self.dim, self.heads, self.causal, self.dropout = dim, heads, causal, dropout
        self.qkv = Linear(dim, 3 * dim)
        self.out = Linear(dim, dim)

    def forward(self, x, key_padding: Optional[torch.Tensor] = None, residual=None):
        N, T, C = x.shape
        D = C // self.heads
        q, k, v = self.qkv(x).view(N, T, 3, self.heads, D).unbind(2)
        if _fast(x) and key_padding is None and D in (64, 128) and not (self.training and self.dropout):
            a = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), self.causal, 1.0 / math.sqrt(D))
        else:
            mask = None
            if key_padding is not None:
                mask = ~key_padding[:, None, None, :]
                if self.causal:
                    mask = mask & torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                               dropout_p=self.dropout if self.training else 0.0,
                                               is_causal=self.causal and mask is None).transpose(1, 2)
        return self.out(a.reshape(N, T, C), residual)


class CrossAttention(nn.Module):
    """Queries from ``x`` ``[N, T, dim]``, keys / values from ``memory`` ``[N, S, memory_dim]``."""

    def __init__(self, dim: int, heads: int, memory_dim: Optional[int] = None):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.q = Linear(dim, dim)
        self.kv = Linear(memory_dim or dim, 2 * dim)
        self.out = Linear(dim, dim)

    def forward(self, x, memory, memory_padding: Optional[torch.Tensor] = None):
        N, T, C = x.shape
        S, D = memory.shape[1], C // self.heads
        q = self.q(x).view(N, T, self.heads, D).transpose(1, 2)
        k, v = self.kv(memory).view(N, S, 2, self.heads, D).unbind(2)
        mask = None if memory_padding is None else ~memory_padding[:, None, None, :]
        a = F.scaled_dot_product_attention(q, k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask)
        return self.out(a.transpose(1, 2).reshape(N, T, C))


class RelativePositionAttention(nn.Module):
    """Self-attention whose scores and outputs also depend on the distance between positions: a learned key vector and
    a learned value vector per relative offset in ``[-window, window]`` (shared by the heads), added to the content
    scores and to the attended values. Offsets beyond the window use the window's edge. ``lengths`` masks padding."""

    def __init__(self, dim: int, heads: int, window: int = 4):
        super().__init__()
        if dim % heads:
            raise ValueError("dim must be a multiple of heads")
        self.dim, self.heads, self.window = dim, heads, window
        d = dim // heads
        self.qkv = Linear(dim, 3 * dim)
        self.out = Linear(dim, dim)
        self.rel_k = nn.Parameter(torch.randn(2 * window + 1, d) * d ** -0.5)
        self.rel_v = nn.Parameter(torch.randn(2 * window + 1, d) * d ** -0.5)

    def forward(self, x, lengths: Optional[torch.Tensor] = None):
        N, T, _ = x.shape
        H, D = self.heads, self.dim // self.heads
        q, k, v = self.qkv(x).float().view(N, T, 3, H, D).permute(2, 0, 3, 1, 4)           # [N, H, T, D] each
        pos = torch.arange(T, device=x.device)
        offset = (pos[None, :] - pos[:, None]).clamp(-self.window, self.window) + self.window   # [T, T]
        rk, rv = self.rel_k.float()[offset], self.rel_v.float()[offset]                       # [T, T, D]
        scores = (q @ k.transpose(-1, -2) + torch.einsum("nhtd,tsd->nhts", q, rk)) * D ** -0.5
        if lengths is not None:
            keep = pos[None, :] < lengths.to(x.device)[:, None]                               # [N, T]
            scores = scores.masked_fill(~keep[:, None, None, :], float("-inf"))
        p = ops_reduce.softmax(scores, -1)
        a = p @ v + torch.einsum("nhts,tsd->nhtd", p, rv)
        return self.out(a.transpose(1, 2).reshape(N, T, self.dim).to(x.dtype))


class WaveNetBlock(nn.Module):
    """A stack of dilated, gated 1-D convolutions over ``[N, channels, T]`` with residual and skip connections and an
    optional conditioning input added before the gate (the body of a flow's coupling network and of neural vocoders)."""

    def __init__(self, channels: int, kernel: int = 5, layers: int = 4, dilation_rate: int = 2, condition: int = 0):
        super().__init__()
        self.channels, self.kernel, self.layers, self.dilation_rate, self.condition = channels, kernel, layers, dilation_rate, condition
        self.dilated = nn.ModuleList()
        self.mix = nn.ModuleList()
        for i in range(layers):
            d = dilation_rate ** i
            self.dilated.append(nn.Conv1d(channels, 2 * channels, kernel, dilation=d, padding=(kernel - 1) * d // 2))
            self.mix.append(nn.Conv1d(channels, 2 * channels if i + 1 < layers else channels, 1))
        self.cond = nn.Conv1d(condition, 2 * channels * layers, 1) if condition else None

    def forward(self, x, condition: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None):
        skip = torch.zeros_like(x)
        g = self.cond(condition) if self.cond is not None and condition is not None else None
        for i in range(self.layers):
            h = self.dilated[i](x)
            if g is not None:
                h = h + g[:, 2 * self.channels * i: 2 * self.channels * (i + 1)]
            a, b = h.chunk(2, 1)
            h = self.mix[i](torch.tanh(a) * torch.sigmoid(b))
            if i + 1 < self.layers:
                r, s = h.chunk(2, 1)
                x = x + r if mask is None else (x + r) * mask
                skip = skip + s
            else:
                skip = skip + h
        return skip if mask is None else skip * mask


class AffineCoupling(nn.Module):
    """One step of a normalising flow over ``[N, channels, T]``: the first half of the channels passes through and
    parameterises (through a WaveNet block) a shift and a log-scale for the second half. ``forward`` returns the
    transformed tensor and the log-determinant per sequence; ``reverse`` inverts it exactly."""

    def __init__(self, channels: int, hidden: int = 64, kernel: int = 5, layers: int = 3, condition: int = 0,
                 mean_only: bool = False):
        super().__init__()
        if channels % 2:
            raise ValueError("a coupling layer splits the channels in two halves")
        self.channels, self.hidden, self.mean_only = channels, hidden, mean_only
        half = channels // 2
        self.pre = nn.Conv1d(half, hidden, 1)
        self.body = WaveNetBlock(hidden, kernel, layers, 1, condition)
        self.post = nn.Conv1d(hidden, half if mean_only else 2 * half, 1)
        nn.init.zeros_(self.post.weight)             # starts as the identity
        nn.init.zeros_(self.post.bias)

    def _stats(self, x0, condition, mask):
        h = self.pre(x0)
        h = self.post(self.body(h if mask is None else h * mask, condition, mask))
        if self.mean_only:
            return h, torch.zeros_like(h)
        shift, log_scale = h.chunk(2, 1)
        return shift, log_scale

    def forward(self, x, condition=None, mask=None):
        x0, x1 = x.chunk(2, 1)
        shift, log_scale = self._stats(x0, condition, mask)
        y1 = shift + x1 * torch.exp(log_scale)
        if mask is not None:
            y1, log_scale = y1 * mask, log_scale * mask
        return torch.cat([x0, y1], 1), log_scale.sum((1, 2))

    def reverse(self, y, condition=None, mask=None):
        y0, y1 = y.chunk(2, 1)
        shift, log_scale = self._stats(y0, condition, mask)
        x1 = (y1 - shift) * torch.exp(-log_scale)
        return torch.cat([y0, x1 if mask is None else x1 * mask], 1)


class TransformerEncoderLayer(nn.Module):
    """Attention + feed-forward with residuals; ``norms`` 'before' (pre-norm) or 'after' (post-norm)."""

    def __init__(self, dim: int, heads: int, ff_dim: int, dropout: float = 0.0, causal: bool = False, norms: str = "before",
                 activation: str = "gelu"):
        super().__init__()
        if norms not in ("before", "after"):
            raise ValueError("norms must be 'before' or 'after'")
        self.dim, self.ff_dim, self.norms, self.activation = dim, ff_dim, norms, activation
        self.norm1 = LayerNorm(dim)
        self.attention = MultiHeadAttention(dim, heads, causal, dropout)
        self.norm2 = LayerNorm(dim)
        self.up = Linear(dim, ff_dim)
        self.down = Linear(ff_dim, dim)
        self.drop = nn.Dropout(dropout)

    def _ff(self, h, residual):
        act = F.gelu if self.activation == "gelu" else F.relu
        return self.down(self.drop(act(self.up(h))), residual)

    def forward(self, x, key_padding: Optional[torch.Tensor] = None):
        if self.norms == "before":
            x = self.attention(self.norm1(x), key_padding, residual=x)
            return self._ff(self.norm2(x), x)
        x = self.norm1(self.attention(x, key_padding, residual=x))
        return self.norm2(self._ff(x, x))


class Conv2d(nn.Conv2d):
    """``nn.Conv2d`` whose CUDA forward and backward run the package's kernels: patch rows around the tcgen05 GEMM for a
    dense bf16 convolution, the depthwise kernel when every channel is its own group (``ops/conv.py``)."""

    def forward(self, x):
        if x.is_cuda and self.padding_mode == "zeros" and not isinstance(self.padding, str):
            return conv_ops.conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)
        return super().forward(x)


class Conv1d(nn.Conv1d):
    def forward(self, x):
        if x.is_cuda and self.padding_mode == "zeros" and not isinstance(self.padding, str):
            return conv_ops.conv1d(x, self.weight, self.bias, self.stride[0], self.padding[0], self.dilation[0],
                                   self.groups)
        return super().forward(x)


class MaxPool2d(nn.MaxPool2d):
    def forward(self, x):
        if x.is_cuda and x.dim() == 4 and not self.return_indices:
            return conv_ops.max_pool2d(x, self.kernel_size, self.stride, self.padding, self.dilation, self.ceil_mode)
        return super().forward(x)


class AvgPool2d(nn.AvgPool2d):
    def forward(self, x):
        if x.is_cuda and x.dim() == 4 and self.divisor_override is None:
            return conv_ops.avg_pool2d(x, self.kernel_size, self.stride, self.padding, self.ceil_mode,
                                       self.count_include_pad)
        return super().forward(x)


class Recurrent(nn.Module):
    """LSTM / GRU over ``[N, T, in]``: all steps (``sequences=True``) or the last step's output."""

    def __init__(self, kind: str, in_features: int, hidden: int, sequences: bool = False, bidirectional: bool = False,
                 layers: int = 1):
        super().__init__()
        self.kind, self.in_features, self.hidden = kind, in_features, hidden
        self.sequences, self.bidirectional, self.layers = sequences, bidirectional, layers
        cls = nn.LSTM if kind == "lstm" else nn.GRU
        self.cell = cls(in_features, hidden, num_layers=layers, batch_first=True, bidirectional=bidirectional)

    def forward(self, x):
        if x.is_cuda:
            out, _ = recurrent_ops.run_module(self.cell, x)       # the package's cell kernels and products
        else:
            out, _ = self.cell(x)
        if self.sequences:
            return out
        if self.bidirectional:
            return torch.cat([out[:, -1, : self.hidden], out[:, 0, self.hidden:]], dim=-1)
        return out[:, -1]


class GlobalAveragePool2d(nn.Module):
    def forward(self, x):
        return x.mean((2, 3))


class QuickGELU(nn.Module):
    def forward(self, x):
        return x * torch.sigmoid(1.702 * x)


class Sequential(nn.Sequential):
    """``nn.Sequential`` that remembers the description it was built from (``architecture``)."""
    architecture: Optional[dict] = None


def weight_norm(module: nn.Module, name: str = "weight") -> nn.Module:
    """Reparameterise ``module.<name>`` as direction x magnitude."""
    return nn.utils.parametrizations.weight_norm(module, name)


# ---------------------------------------------------------------------------------------------------------------------
# layer types: name -> (describe(module) -> dict of fields, create(fields) -> module)
# ---------------------------------------------------------------------------------------------------------------------
def _pair(v) -> Tuple[int, int]:
    return (int(v[0]), int(v[1])) if isinstance(v, (list, tuple)) else (int(v), int(v))


def _defaults(t: SlotTable) -> None:
    def reg(name: str, cls, describe: Callable, create: Callable):
        t.register(name, (cls, describe, create), "fallback")

    reg("linear", Linear, lambda m: {"in": m.in_features, "out": m.out_features, "bias": m.bias is not None},
        lambda d: Linear(d["in"], d["out"], d.get("bias", True)))
    reg("embedding", Embedding, lambda m: {"vocabulary": m.vocabulary, "dim": m.dim}, lambda d: Embedding(d["vocabulary"], d["dim"]))
    reg("layernorm", LayerNorm, lambda m: {"features": m.features, "epsilon": m.epsilon},
        lambda d: LayerNorm(d["features"], d.get("epsilon", 1e-5)))
    reg("rmsnorm", RMSNorm, lambda m: {"features": m.features, "epsilon": m.epsilon},
        lambda d: RMSNorm(d["features"], d.get("epsilon", 1e-6)))
    reg("positional", PositionalEncoding, lambda m: {"maxLength": m.max_length, "dim": m.dim},
        lambda d: PositionalEncoding(d["maxLength"], d["dim"]))
    reg("attention", MultiHeadAttention, lambda m: {"dim": m.dim, "heads": m.heads, "causal": m.causal},
        lambda d: MultiHeadAttention(d["dim"], d["heads"], d.get("causal", False)))
    reg("transformer", TransformerEncoderLayer,
        lambda m: {"dim": m.dim, "heads": m.attention.heads, "ffDim": m.ff_dim, "causal": m.attention.causal,
                   **({"norms": "after"} if m.norms == "after" else {})},
        lambda d: TransformerEncoderLayer(d["dim"], d["heads"], d["ffDim"], 0.0, d.get("causal", False), d.get("norms", "before")))
    reg("relative_attention", RelativePositionAttention, lambda m: {"dim": m.dim, "heads": m.heads, "window": m.window},
        lambda d: RelativePositionAttention(d["dim"], d["heads"], d.get("window", 4)))
    reg("wavenet", WaveNetBlock,
        lambda m: {"channels": m.channels, "kernel": m.kernel, "layers": m.layers, "dilationRate": m.dilation_rate,
                   **({"condition": m.condition} if m.condition else {})},
        lambda d: WaveNetBlock(d["channels"], d.get("kernel", 5), d.get("layers", 4), d.get("dilationRate", 2), d.get("condition", 0)))
    reg("affine_coupling", AffineCoupling,
        lambda m: {"channels": m.channels, "hidden": m.hidden, "kernel": m.body.kernel, "layers": m.body.layers,
                   **({"condition": m.body.condition} if m.body.condition else {}), **({"meanOnly": True} if m.mean_only else {})},
        lambda d: AffineCoupling(d["channels"], d.get("hidden", 64), d.get("kernel", 5), d.get("layers", 3), d.get("condition", 0),
                                 d.get("meanOnly", False)))
    for kind in ("lstm", "gru"):
        reg(kind, None, lambda m: {"in": m.in_features, "hidden": m.hidden, "sequences": m.sequences,
                                   **({"bidirectional": True} if m.bidirectional else {}),
                                   **({"layers": m.layers} if m.layers != 1 else {})},
            lambda d, kind=kind: Recurrent(kind, d["in"], d["hidden"], d.get("sequences", False), d.get("bidirectional", False),
                                           d.get("layers", 1)))
    reg("conv2d", nn.Conv2d,
        lambda m: {"in": m.in_channels, "out": m.out_channels, "kernel": list(m.kernel_size), "stride": list(m.stride),
                   "padding": list(m.padding), "bias": m.bias is not None,
                   **({"dilation": list(m.dilation)} if tuple(m.dilation) != (1, 1) else {}),
                   **({"groups": m.groups} if m.groups != 1 else {})},
        lambda d: Conv2d(d["in"], d["out"], _pair(d["kernel"]), _pair(d.get("stride", 1)), _pair(d.get("padding", 0)),
                            _pair(d.get("dilation", 1)), d.get("groups", 1), d.get("bias", True)))
    reg("conv1d", nn.Conv1d,
        lambda m: {"in": m.in_channels, "out": m.out_channels, "kernel": m.kernel_size[0], "stride": m.stride[0],
                   "padding": m.padding[0], "bias": m.bias is not None},
        lambda d: Conv1d(d["in"], d["out"], d["kernel"], d.get("stride", 1), d.get("padding", 0), bias=d.get("bias", True)))
    reg("convtranspose2d", nn.ConvTranspose2d,
        lambda m: {"in": m.in_channels, "out": m.out_channels, "kernel": list(m.kernel_size), "stride": list(m.stride),
                   "padding": list(m.padding), "outputPadding": list(m.output_padding), "dilation": list(m.dilation),
                   "groups": m.groups, "bias": m.bias is not None},
        lambda d: nn.ConvTranspose2d(d["in"], d["out"], _pair(d["kernel"]), _pair(d.get("stride", 1)), _pair(d.get("padding", 0)),
                                     _pair(d.get("outputPadding", 0)), d.get("groups", 1), d.get("bias", True),
                                     _pair(d.get("dilation", 1))))
    reg("batchnorm", nn.BatchNorm2d, lambda m: {"channels": m.num_features, "momentum": m.momentum, "epsilon": m.eps},
        lambda d: nn.BatchNorm2d(d["channels"], d.get("epsilon", 1e-5), d.get("momentum", 0.1)))
    reg("groupnorm", nn.GroupNorm, lambda m: {"groups": m.num_groups, "channels": m.num_channels, "epsilon": m.eps, "affine": m.affine},
        lambda d: nn.GroupNorm(d["groups"], d["channels"], d.get("epsilon", 1e-5), d.get("affine", True)))
    reg("maxpool2d", nn.MaxPool2d,
        lambda m: {"kernel": list(_pair(m.kernel_size)), "stride": list(_pair(m.stride)), "padding": list(_pair(m.padding)),
                   **({"ceilMode": True} if m.ceil_mode else {})},
        lambda d: MaxPool2d(_pair(d["kernel"]), _pair(d.get("stride", d["kernel"])), _pair(d.get("padding", 0)),
                               ceil_mode=d.get("ceilMode", False)))
    reg("avgpool2d", nn.AvgPool2d,
        lambda m: {"kernel": list(_pair(m.kernel_size)), "stride": list(_pair(m.stride)), "padding": list(_pair(m.padding)),
                   "countIncludePad": m.count_include_pad, **({"ceilMode": True} if m.ceil_mode else {})},
        lambda d: AvgPool2d(_pair(d["kernel"]), _pair(d.get("stride", d["kernel"])), _pair(d.get("padding", 0)),
                               d.get("ceilMode", False), d.get("countIncludePad", True)))
    reg("adaptiveavgpool2d", nn.AdaptiveAvgPool2d, lambda m: {"size": list(_pair(m.output_size))},
        lambda d: nn.AdaptiveAvgPool2d(_pair(d["size"])))
    reg("adaptivemaxpool2d", nn.AdaptiveMaxPool2d, lambda m: {"size": list(_pair(m.output_size))},
        lambda d: nn.AdaptiveMaxPool2d(_pair(d["size"])))
    reg("upsample", nn.Upsample,
        lambda m: {**({"size": list(_pair(m.size))} if m.size is not None else {"scale": list(map(float, _scale(m.scale_factor)))}),
                   "mode": m.mode, "alignCorners": bool(m.align_corners)},
        lambda d: nn.Upsample(size=_pair(d["size"]) if "size" in d else None,
                              scale_factor=tuple(d["scale"]) if "scale" in d else None, mode=d.get("mode", "nearest"),
                              align_corners=(d.get("alignCorners", False) if d.get("mode") == "bilinear" else None)))
    reg("globalavgpool2d", GlobalAveragePool2d, lambda m: {}, lambda d: GlobalAveragePool2d())
    reg("flatten", nn.Flatten, lambda m: {}, lambda d: nn.Flatten())
    reg("relu", nn.ReLU, lambda m: {}, lambda d: nn.ReLU())
    reg("tanh", nn.Tanh, lambda m: {}, lambda d: nn.Tanh())
    reg("sigmoid", nn.Sigmoid, lambda m: {}, lambda d: nn.Sigmoid())
    reg("gelu", nn.GELU, lambda m: {}, lambda d: nn.GELU(approximate="tanh"))
    reg("gelu_exact", None, lambda m: {}, lambda d: nn.GELU())
    reg("quick_gelu", QuickGELU, lambda m: {}, lambda d: QuickGELU())
    reg("softmax", nn.Softmax, lambda m: {}, lambda d: nn.Softmax(dim=-1))
    reg("dropout", nn.Dropout, lambda m: {"p": m.p}, lambda d: nn.Dropout(d.get("p", 0.5)))
    reg("sequential", Sequential,
        lambda m: {"network": m.architecture} if getattr(m, "architecture", None) else {"layers": [describe(c) for c in m]},
        lambda d: _sequential(d))


def _scale(v):
    return v if isinstance(v, (list, tuple)) else (v, v)


def _sequential(d: dict) -> Sequential:
    if "network" in d:
        from .builder import Network
        return Network.from_json(d["network"]).build()
    return Sequential(*[create(layer) for layer in d["layers"]])


LAYER_TYPES: SlotTable = SlotTable("layer types", _defaults)


def type_name(module: nn.Module) -> str:
    if isinstance(module, Recurrent):
        return module.kind
    if isinstance(module, nn.GELU):
        return "gelu" if module.approximate == "tanh" else "gelu_exact"
    for name, (cls, _, _) in LAYER_TYPES.items():
        if cls is not None and type(module) is cls:
            return name
    for name, (cls, _, _) in LAYER_TYPES.items():
        if cls is not None and isinstance(module, cls):
            return name
    raise KeyError(f"no layer type describes {type(module).__name__}; register one in LAYER_TYPES")


def describe(module: nn.Module) -> dict:
    name = type_name(module)
    return {"type": name, **LAYER_TYPES[name][1](module)}


def create(description: dict) -> nn.Module:
    d = dict(description)
    name = d.pop("type")
    return LAYER_TYPES[name][2](d)
