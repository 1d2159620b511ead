"""Vision transformer for image classification and image embeddings, on the same kernels as the decoder:
the fused resize + normalise preprocessing, GEMM projections with fused epilogues and LayerNorm (attention over the
197 patch rows goes to the library's scaled-dot-product attention on CUDA). Loads Hugging Face ViT checkpoints (``vit.*`` tensor names).

Reference: the vision package of the reference (src/Idrak.Vision: ViT encoder, image classifier, preprocessing
pipeline) - here as a thin model over this package's ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from ..ops.image import resize_normalize


@dataclass
class VitSpec:
    image_size: int = 224
    patch_size: int = 16
    channels: int = 3
    dim: int = 768
    layers: int = 12
    heads: int = 12
    ff_dim: int = 3072
    classes: int = 1000
    norm_epsilon: float = 1e-12
    mean: Tuple[float, ...] = (0.5, 0.5, 0.5)
    std: Tuple[float, ...] = (0.5, 0.5, 0.5)

    @property
    def patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @classmethod
    def from_hf_config(cls, cfg: dict) -> "VitSpec":
        return cls(image_size=cfg.get("image_size", 224), patch_size=cfg.get("patch_size", 16),
                   channels=cfg.get("num_channels", 3), dim=cfg["hidden_size"], layers=cfg["num_hidden_layers"],
                   heads=cfg["num_attention_heads"], ff_dim=cfg["intermediate_size"],
                   classes=len(cfg.get("id2label", {})) or cfg.get("num_labels", 2),
                   norm_epsilon=cfg.get("layer_norm_eps", 1e-12))


class VitBlock(nn.Module):
    def __init__(self, s: VitSpec):
        super().__init__()
        self.s = s
        self.norm1_w, self.norm1_b = nn.Parameter(torch.ones(s.dim)), nn.Parameter(torch.zeros(s.dim))
        self.qkv_w, self.qkv_b = nn.Parameter(torch.empty(3 * s.dim, s.dim)), nn.Parameter(torch.zeros(3 * s.dim))
        self.o_w, self.o_b = nn.Parameter(torch.empty(s.dim, s.dim)), nn.Parameter(torch.zeros(s.dim))
        self.norm2_w, self.norm2_b = nn.Parameter(torch.ones(s.dim)), nn.Parameter(torch.zeros(s.dim))
        self.up_w, self.up_b = nn.Parameter(torch.empty(s.ff_dim, s.dim)), nn.Parameter(torch.zeros(s.ff_dim))
        self.down_w, self.down_b = nn.Parameter(torch.empty(s.dim, s.ff_dim)), nn.Parameter(torch.zeros(s.dim))

    def forward(self, x):
        s = self.s
        B, T, C = x.shape
        D = C // s.heads
        h = ops.layer_norm(x, self.norm1_w, self.norm1_b, s.norm_epsilon)
        qkv = ops.linear(h, self.qkv_w, self.qkv_b).view(B, T, 3, s.heads, D)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if x.is_cuda:
            # 1 + patches rows (197) is not a tile multiple and the mask is full: the library's attention serves here
            a = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                 scale=1.0 / math.sqrt(D)).transpose(1, 2)
        else:
            a = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), False, 1.0 / math.sqrt(D))
        x = ops.linear(a.reshape(B, T, C).contiguous(), self.o_w, self.o_b, x)
        h = ops.layer_norm(x, self.norm2_w, self.norm2_b, s.norm_epsilon)
        h = torch.nn.functional.gelu(ops.linear(h, self.up_w, self.up_b))      # ViT uses the exact (erf) GELU
        return ops.linear(h, self.down_w, self.down_b, x)


class VisionTransformer(nn.Module):
    def __init__(self, spec: VitSpec):
        super().__init__()
        self.spec = s = spec
        patch_in = s.channels * s.patch_size * s.patch_size
        self.patch_w, self.patch_b = nn.Parameter(torch.empty(s.dim, patch_in)), nn.Parameter(torch.zeros(s.dim))
        self.cls = nn.Parameter(torch.zeros(1, 1, s.dim))
        self.pos = nn.Parameter(torch.zeros(1, s.patches + 1, s.dim))
        self.blocks = nn.ModuleList([VitBlock(s) for _ in range(s.layers)])
        self.norm_w, self.norm_b = nn.Parameter(torch.ones(s.dim)), nn.Parameter(torch.zeros(s.dim))
        self.head_w, self.head_b = nn.Parameter(torch.empty(s.classes, s.dim)), nn.Parameter(torch.zeros(s.classes))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: Optional[int] = None):
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        for p in self.parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)

    def preprocess(self, images: torch.Tensor) -> torch.Tensor:
        """uint8 ``[N, H, W, C]`` -> normalised ``[N, C, S, S]`` in the model's dtype (one fused kernel on CUDA)."""
        s = self.spec
        dtype = self.patch_w.dtype if self.patch_w.dtype in (torch.float32, torch.bfloat16) else torch.float32
        return resize_normalize(images.to(self.patch_w.device), (s.image_size, s.image_size), s.mean, s.std, "bilinear", dtype)

    def hidden(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[N, C, S, S]`` pixels -> final hidden states ``[N, 1 + patches, dim]`` (class token first)."""
        s = self.spec
        N = pixels.shape[0]
        P = s.patch_size
        g = s.image_size // P
        # [N, C, g, P, g, P] -> [N, g, g, C, P, P]: one row per patch in (channel, y, x) order, as a Conv2d kernel sees it
        patches = pixels.view(N, s.channels, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(N, g * g, -1)
        x = ops.linear(patches.contiguous().to(self.patch_w.dtype), self.patch_w, self.patch_b)
        x = torch.cat([self.cls.expand(N, -1, -1).to(x.dtype), x], dim=1) + self.pos.to(x.dtype)
        for blk in self.blocks:
            x = blk(x)
        return ops.layer_norm(x, self.norm_w, self.norm_b, s.norm_epsilon)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """Class logits ``[N, classes]``."""
        h = self.hidden(pixels)
        return ops.linear(h[:, 0].contiguous(), self.head_w, self.head_b)

    def embed(self, pixels: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.normalize(self.hidden(pixels)[:, 0].float(), dim=-1)

    # ------------------------------------------------------------------ Hugging Face names
    def load_hf_tensors(self, src: Mapping[str, torch.Tensor]) -> None:
        s = self.spec

        def get(name):
            for prefix in ("vit.", ""):
                if prefix + name in src:
                    return src[prefix + name]
            raise KeyError(f"the checkpoint has no tensor '{name}'")

        with torch.no_grad():
            self.patch_w.copy_(get("embeddings.patch_embeddings.projection.weight").reshape(s.dim, -1))
            self.patch_b.copy_(get("embeddings.patch_embeddings.projection.bias"))
            self.cls.copy_(get("embeddings.cls_token"))
            self.pos.copy_(get("embeddings.position_embeddings"))
            for i, b in enumerate(self.blocks):
                p = f"encoder.layer.{i}."
                b.norm1_w.copy_(get(p + "layernorm_before.weight")); b.norm1_b.copy_(get(p + "layernorm_before.bias"))
                b.norm2_w.copy_(get(p + "layernorm_after.weight")); b.norm2_b.copy_(get(p + "layernorm_after.bias"))
                b.qkv_w.copy_(torch.cat([get(p + f"attention.attention.{n}.weight") for n in ("query", "key", "value")]))
                b.qkv_b.copy_(torch.cat([get(p + f"attention.attention.{n}.bias") for n in ("query", "key", "value")]))
                b.o_w.copy_(get(p + "attention.output.dense.weight")); b.o_b.copy_(get(p + "attention.output.dense.bias"))
                b.up_w.copy_(get(p + "intermediate.dense.weight")); b.up_b.copy_(get(p + "intermediate.dense.bias"))
                b.down_w.copy_(get(p + "output.dense.weight")); b.down_b.copy_(get(p + "output.dense.bias"))
            self.norm_w.copy_(get("layernorm.weight")); self.norm_b.copy_(get("layernorm.bias"))
            if "classifier.weight" in src:
                self.head_w.copy_(src["classifier.weight"]); self.head_b.copy_(src["classifier.bias"])


class ImageClassifier:
    """Images in, labels out: preprocessing, the model, soft-max, top-k."""

    def __init__(self, model: VisionTransformer, labels: Optional[Sequence[str]] = None):
        self.model, self.labels = model.eval(), list(labels) if labels else None

    @torch.no_grad()
    def classify(self, images: torch.Tensor, k: int = 5):
        logits = self.model(self.model.preprocess(images)).float()
        probs = torch.softmax(logits, -1)
        top = torch.topk(probs, min(k, probs.shape[-1]))
        out = []
        for row_p, row_i in zip(top.values.tolist(), top.indices.tolist()):
            out.append([{"label": self.labels[i] if self.labels else str(i), "index": i, "probability": p}
                        for p, i in zip(row_p, row_i)])
        return out
