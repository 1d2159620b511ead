"""Detection utilities: box arithmetic, non-maximum suppression, box-aware augmentations and the COCO / VOC
mean-average-precision metrics.

Boxes are ``[x0, y0, x1, y1]`` in pixels (float tensors ``[n, 4]``). Everything runs on the device of its inputs.

Reference: src/Idrak.Vision (Boxes, NonMaximumSuppression, DetectionMetrics with COCO 101-point and VOC all-point
interpolation, augmentations that carry boxes along).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------------------------------
# boxes
# ---------------------------------------------------------------------------------------------------------------------
def box_area(b: torch.Tensor) -> torch.Tensor:
    return (b[..., 2] - b[..., 0]).clamp_min(0) * (b[..., 3] - b[..., 1]).clamp_min(0)


def box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Pairwise intersection over union ``[len(a), len(b)]``."""
    lt = torch.maximum(a[:, None, :2], b[None, :, :2])
    rb = torch.minimum(a[:, None, 2:], b[None, :, 2:])
    inter = (rb - lt).clamp_min(0).prod(-1)
    union = box_area(a)[:, None] + box_area(b)[None] - inter
    return inter / union.clamp_min(1e-12)


def xywh_to_xyxy(b: torch.Tensor) -> torch.Tensor:
    return torch.cat([b[..., :2], b[..., :2] + b[..., 2:]], -1)


def cxcywh_to_xyxy(b: torch.Tensor) -> torch.Tensor:
    half = b[..., 2:] / 2
    return torch.cat([b[..., :2] - half, b[..., :2] + half], -1)


def nms(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float = 0.5, classes: Optional[torch.Tensor] = None,
        top_k: int = 0) -> torch.Tensor:
    """Indices kept, best score first. With ``classes`` boxes only suppress boxes of their own class."""
    if boxes.numel() == 0:
        return torch.zeros(0, dtype=torch.long, device=boxes.device)
    order = scores.argsort(descending=True)
    b = boxes[order].float()
    if classes is not None:
        # shift every class to its own region of the plane so different classes never overlap
        span = b.max() + 1
        b = b + (classes[order].float() * span)[:, None]
    iou = box_iou(b, b)
    n = len(order)
    suppressed = torch.zeros(n, dtype=torch.bool, device=boxes.device)
    keep = []
    over = iou > iou_threshold
    for i in range(n):
        if suppressed[i]:
            continue
        keep.append(i)
        if top_k and len(keep) >= top_k:
            break
        suppressed |= over[i]
    return order[torch.tensor(keep, dtype=torch.long, device=boxes.device)]


# ---------------------------------------------------------------------------------------------------------------------
# augmentations that carry boxes
# ---------------------------------------------------------------------------------------------------------------------
def flip_horizontal(image: torch.Tensor, boxes: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``image`` [..., H, W, C] or [..., C, H, W] given as channels-last here: [H, W, C]."""
    W = image.shape[1]
    out = boxes.clone()
    out[:, 0], out[:, 2] = W - boxes[:, 2], W - boxes[:, 0]
    return image.flip(1), out


def crop(image: torch.Tensor, boxes: torch.Tensor, window: Tuple[int, int, int, int], min_visible: float = 0.3):
    """Crop ``[H, W, C]`` to ``window = (x0, y0, x1, y1)``; boxes are clipped, and dropped when less than ``min_visible``
    of their area stays inside. Returns (image, boxes, kept indices)."""
    x0, y0, x1, y1 = window
    shifted = boxes - torch.tensor([x0, y0, x0, y0], dtype=boxes.dtype, device=boxes.device)
    clipped = torch.stack([shifted[:, 0].clamp(0, x1 - x0), shifted[:, 1].clamp(0, y1 - y0),
                           shifted[:, 2].clamp(0, x1 - x0), shifted[:, 3].clamp(0, y1 - y0)], 1)
    keep = (box_area(clipped) >= min_visible * box_area(boxes).clamp_min(1e-9)).nonzero()[:, 0]
    return image[y0:y1, x0:x1], clipped[keep], keep


def random_crop(image, boxes, rng: np.random.Generator, scale: Tuple[float, float] = (0.5, 1.0), min_visible: float = 0.3):
    H, W = image.shape[:2]
    s = float(rng.uniform(*scale))
    h, w = max(int(H * s), 1), max(int(W * s), 1)
    y0, x0 = int(rng.integers(0, H - h + 1)), int(rng.integers(0, W - w + 1))
    return crop(image, boxes, (x0, y0, x0 + w, y0 + h), min_visible)


def resize_boxes(boxes: torch.Tensor, from_size: Tuple[int, int], to_size: Tuple[int, int]) -> torch.Tensor:
    sy, sx = to_size[0] / from_size[0], to_size[1] / from_size[1]
    return boxes * torch.tensor([sx, sy, sx, sy], dtype=boxes.dtype, device=boxes.device)


def color_jitter(image: torch.Tensor, rng: np.random.Generator, brightness: float = 0.2, contrast: float = 0.2,
                 saturation: float = 0.2) -> torch.Tensor:
    """uint8 ``[H, W, 3]`` -> jittered uint8."""
    x = image.float()
    x = x * float(1 + rng.uniform(-brightness, brightness))
    mean = x.mean()
    x = (x - mean) * float(1 + rng.uniform(-contrast, contrast)) + mean
    grey = x.mean(-1, keepdim=True)
    x = (x - grey) * float(1 + rng.uniform(-saturation, saturation)) + grey
    return x.round().clamp(0, 255).to(torch.uint8)


# ---------------------------------------------------------------------------------------------------------------------
# mean average precision
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Detections:
    boxes: torch.Tensor           # [n, 4]
    scores: torch.Tensor          # [n]
    labels: torch.Tensor          # [n]


@dataclass
class GroundTruth:
    boxes: torch.Tensor           # [m, 4]
    labels: torch.Tensor          # [m]
    crowd: Optional[torch.Tensor] = None     # [m] bool: matches to these neither count nor hurt


def _average_precision(recall: np.ndarray, precision: np.ndarray, style: str) -> float:
    # precision envelope (monotone from the right)
    mrec = np.concatenate([[0.0], recall, [1.0]])
    mpre = np.concatenate([[0.0], precision, [0.0]])
    for i in range(len(mpre) - 2, -1, -1):
        mpre[i] = max(mpre[i], mpre[i + 1])
    if style == "coco":                                  # 101 recall points
        points = np.linspace(0, 1, 101)
        idx = np.searchsorted(mrec, points, side="left")
        return float(np.mean([mpre[i] if i < len(mpre) else 0.0 for i in idx]))
    if style == "voc07":                                 # 11 points
        return float(np.mean([mpre[mrec >= t].max() if (mrec >= t).any() else 0.0 for t in np.linspace(0, 1, 11)]))
    step = np.nonzero(mrec[1:] != mrec[:-1])[0]          # all points (VOC 2010+)
    return float(np.sum((mrec[step + 1] - mrec[step]) * mpre[step + 1]))


def average_precision(detections: Sequence[Detections], truths: Sequence[GroundTruth], label: int, iou_threshold: float = 0.5,
                      style: str = "coco") -> Optional[float]:
    """AP of one class over a set of images (None when the class has no ground truth)."""
    records = []                                          # (score, is true positive)
    total = 0
    for det, gt in zip(detections, truths):
        gsel = (gt.labels == label).nonzero()[:, 0]
        crowd = gt.crowd[gsel] if gt.crowd is not None else torch.zeros(len(gsel), dtype=torch.bool)
        total += int((~crowd).sum())
        dsel = (det.labels == label).nonzero()[:, 0]
        if len(dsel) == 0:
            continue
        order = det.scores[dsel].argsort(descending=True)
        dsel = dsel[order]
        iou = box_iou(det.boxes[dsel].float(), gt.boxes[gsel].float()) if len(gsel) else torch.zeros(len(dsel), 0)
        taken = torch.zeros(len(gsel), dtype=torch.bool)
        for i in range(len(dsel)):
            best, best_j = iou_threshold, -1
            for j in range(len(gsel)):
                if taken[j] and not crowd[j]:
                    continue
                if best_j >= 0 and not crowd[best_j] and crowd[j]:
                    continue                               # a real match beats a crowd match
                if iou[i, j] >= best:
                    best, best_j = float(iou[i, j]), j
            if best_j >= 0 and crowd[best_j]:
                continue                                   # ignored
            if best_j >= 0:
                taken[best_j] = True
            records.append((float(det.scores[dsel[i]]), best_j >= 0))
    if total == 0:
        return None
    if not records:
        return 0.0
    records.sort(key=lambda r: -r[0])
    tp = np.cumsum([r[1] for r in records])
    fp = np.cumsum([not r[1] for r in records])
    return _average_precision(tp / total, tp / np.maximum(tp + fp, 1e-12), style)


def mean_average_precision(detections: Sequence[Detections], truths: Sequence[GroundTruth],
                           iou_thresholds: Sequence[float] = tuple(np.arange(0.5, 0.96, 0.05).round(2)),
                           style: str = "coco") -> Dict[str, float]:
    """COCO-style summary: ``map`` (mean over classes and IoU thresholds), ``map50``, ``map75`` and per-class AP@[.5:.95]."""
    labels = sorted({int(v) for gt in truths for v in gt.labels.tolist()})
    per_class: Dict[int, List[float]] = {}
    for c in labels:
        aps = [average_precision(detections, truths, c, float(t), style) for t in iou_thresholds]
        if aps[0] is not None:
            per_class[c] = [a for a in aps]
    if not per_class:
        return {"map": 0.0, "map50": 0.0, "map75": 0.0}
    ts = [round(float(t), 2) for t in iou_thresholds]
    mean_at = lambda t: float(np.mean([v[ts.index(t)] for v in per_class.values()])) if t in ts else float("nan")
    out = {"map": float(np.mean([np.mean(v) for v in per_class.values()])), "map50": mean_at(0.5), "map75": mean_at(0.75)}
    out.update({f"ap_class_{c}": float(np.mean(v)) for c, v in per_class.items()})
    return out
