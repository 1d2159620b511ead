"""Detection and segmentation models on the package's convolution layers.

``CenterDetector``: an anchor-free detector. A small convolutional backbone reduces the image by four; three heads give,
per cell, a class heat map (a peak where an object's centre is), the object's width and height, and the sub-cell offset
of the centre. Training: penalty-reduced focal loss on the heat map against Gaussian targets, L1 on size and offset at
the centre cells. Decoding: cells that are the maximum of their 3 x 3 neighbourhood (a max pool, so no box-level
suppression is needed) and exceed a threshold become boxes.

``Segmenter``: a small U-shaped network (two reductions, skip connections) that gives class scores per pixel; cross
entropy plus a soft Dice term; ``mean_iou`` scores it.

On a GPU in bf16 the convolutions run as patch rows around the tensor-core GEMM and the pools on the package's kernels
(``nn.layers.Conv2d`` / ``MaxPool2d``).

Reference: the detectors and segmenters of the vision package (src/Idrak.Vision: detector heads, box decoding,
segmentation losses and metrics).
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..nn import layers as L
from .detection import Detections, GroundTruth


def _block(cin: int, cout: int) -> nn.Sequential:
    return nn.Sequential(L.Conv2d(cin, cout, 3, padding=1), nn.BatchNorm2d(cout), nn.ReLU(),
                         L.Conv2d(cout, cout, 3, padding=1), nn.BatchNorm2d(cout), nn.ReLU())


class CenterDetector(nn.Module):
    STRIDE = 4

    def __init__(self, classes: int, channels: int = 3, width: int = 32):
        super().__init__()
        self.classes = classes
        self.backbone = nn.Sequential(_block(channels, width), L.MaxPool2d(2), _block(width, 2 * width), L.MaxPool2d(2),
                                      _block(2 * width, 2 * width))
        def head(out):
            return nn.Sequential(L.Conv2d(2 * width, width, 3, padding=1), nn.ReLU(), L.Conv2d(width, out, 1))
        self.heat, self.size, self.offset = head(classes), head(2), head(2)
        nn.init.constant_(self.heat[-1].bias, -math.log(99.0))        # every cell starts as "1 % object"

    def forward(self, images: torch.Tensor):
        f = self.backbone(images)
        return self.heat(f), self.size(f), self.offset(f)

    # ------------------------------------------------------------------ training
    def targets(self, truths: Sequence[GroundTruth], height: int, width: int, device=None):
        """Heat map ``[N, K, h, w]`` with a Gaussian around every object's centre cell, and per object its image index,
        cell, class, size (in cells) and offset."""
        h, w = height // self.STRIDE, width // self.STRIDE
        heat = torch.zeros(len(truths), self.classes, h, w)
        rows = []
        ys, xs = torch.meshgrid(torch.arange(h).float(), torch.arange(w).float(), indexing="ij")
        for n, gt in enumerate(truths):
            for box, label in zip(gt.boxes.tolist(), gt.labels.tolist()):
                cx, cy = (box[0] + box[2]) / 2 / self.STRIDE, (box[1] + box[3]) / 2 / self.STRIDE
                bw, bh = (box[2] - box[0]) / self.STRIDE, (box[3] - box[1]) / self.STRIDE
                ix, iy = min(int(cx), w - 1), min(int(cy), h - 1)
                sigma = max(min(bw, bh) / 6.0, 0.7)
                g = torch.exp(-((xs - ix) ** 2 + (ys - iy) ** 2) / (2 * sigma * sigma))
                heat[n, int(label)] = torch.maximum(heat[n, int(label)], g)
                rows.append((n, iy, ix, int(label), bw, bh, cx - ix, cy - iy))
        t = torch.tensor(rows, dtype=torch.float32) if rows else torch.zeros(0, 8)
        return heat.to(device), t.to(device)

    def loss(self, outputs, truths: Sequence[GroundTruth], height: int, width: int) -> torch.Tensor:
        heat_logits, size, offset = (o.float() for o in outputs)
        target, rows = self.targets(truths, height, width, heat_logits.device)
        p = torch.sigmoid(heat_logits).clamp(1e-4, 1 - 1e-4)
        positive = target.eq(1.0)
        focal = -(positive * (1 - p) ** 2 * torch.log(p) + (~positive) * (1 - target) ** 4 * p ** 2 * torch.log(1 - p)).sum()
        count = max(len(rows), 1)
        if len(rows) == 0:
            return focal / count
        n, iy, ix = rows[:, 0].long(), rows[:, 1].long(), rows[:, 2].long()
        l1 = (size[n, :, iy, ix] - rows[:, 4:6]).abs().sum() * 0.1 + (offset[n, :, iy, ix] - rows[:, 6:8]).abs().sum()
        return (focal + l1) / count

    # ------------------------------------------------------------------ inference
    @torch.no_grad()
    def detect(self, images: torch.Tensor, threshold: float = 0.3, top_k: int = 50) -> List[Detections]:
        heat_logits, size, offset = (o.float() for o in self(images))
        p = torch.sigmoid(heat_logits)
        peaks = p * (p == F.max_pool2d(p, 3, 1, 1))
        N, K, h, w = p.shape
        out = []
        for n in range(N):
            scores, idx = peaks[n].reshape(-1).topk(min(top_k, K * h * w))
            keep = scores > threshold
            scores, idx = scores[keep], idx[keep]
            label, cell = idx // (h * w), idx % (h * w)
            iy, ix = cell // w, cell % w
            cx = (ix + offset[n, 0, iy, ix]) * self.STRIDE
            cy = (iy + offset[n, 1, iy, ix]) * self.STRIDE
            bw, bh = size[n, 0, iy, ix] * self.STRIDE, size[n, 1, iy, ix] * self.STRIDE
            boxes = torch.stack([cx - bw / 2, cy - bh / 2, cx + bw / 2, cy + bh / 2], 1)
            out.append(Detections(boxes.cpu(), scores.cpu(), label.cpu()))
        return out


class Segmenter(nn.Module):
    def __init__(self, classes: int, channels: int = 3, width: int = 16):
        super().__init__()
        self.classes = classes
        self.down1, self.down2, self.bottom = _block(channels, width), _block(width, 2 * width), _block(2 * width, 4 * width)
        self.pool = L.MaxPool2d(2)
        self.up2, self.up1 = _block(4 * width + 2 * width, 2 * width), _block(2 * width + width, width)
        self.head = L.Conv2d(width, classes, 1)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        d1 = self.down1(images)
        d2 = self.down2(self.pool(d1))
        b = self.bottom(self.pool(d2))
        u2 = self.up2(torch.cat([F.interpolate(b, size=d2.shape[-2:], mode="nearest"), d2], 1))
        u1 = self.up1(torch.cat([F.interpolate(u2, size=d1.shape[-2:], mode="nearest"), d1], 1))
        return self.head(u1)

    def loss(self, logits: torch.Tensor, masks: torch.Tensor, dice_weight: float = 0.5) -> torch.Tensor:
        logits = logits.float()
        ce = F.cross_entropy(logits, masks.long())
        p = torch.softmax(logits, 1)
        onehot = F.one_hot(masks.long(), self.classes).permute(0, 3, 1, 2).float()
        inter = (p * onehot).sum((0, 2, 3))
        dice = 1 - (2 * inter + 1) / (p.sum((0, 2, 3)) + onehot.sum((0, 2, 3)) + 1)
        return ce + dice_weight * dice.mean()


def mean_iou(predicted: torch.Tensor, masks: torch.Tensor, classes: int) -> Tuple[float, List[float]]:
    """Mean intersection over union over the classes present in either, and the per-class values (NaN when absent)."""
    per = []
    for c in range(classes):
        a, b = predicted == c, masks == c
        union = int((a | b).sum())
        per.append(float("nan") if union == 0 else int((a & b).sum()) / union)
    present = [v for v in per if v == v]
    return (sum(present) / len(present) if present else 0.0), per
