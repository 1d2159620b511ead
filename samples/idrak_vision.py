"""Object detection and segmentation on synthetic scenes: 48 x 48 images with one to three filled shapes (disc, square,
triangle) on a noisy background. The anchor-free detector learns boxes and classes (scored with COCO-style mean average
precision); the U-shaped segmenter learns a class per pixel (scored with mean intersection over union).

    python samples/idrak_vision.py [--device cuda]

Reference: samples/IdrakVision.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.vision import CenterDetector, Segmenter, mean_iou  # noqa: E402
from idrak_b200.vision.detection import GroundTruth, mean_average_precision  # noqa: E402

SIZE, CLASSES = 48, 3


def scene(g: torch.Generator):
    """Image [1, S, S], boxes, labels and the per-pixel class mask (0 = background, k + 1 = shape k)."""
    img = 0.1 * torch.rand(SIZE, SIZE, generator=g)
    mask = torch.zeros(SIZE, SIZE, dtype=torch.long)
    ys, xs = torch.meshgrid(torch.arange(SIZE).float(), torch.arange(SIZE).float(), indexing="ij")
    boxes, labels = [], []
    for _ in range(int(torch.randint(1, 4, (), generator=g))):
        r = 4 + 5 * torch.rand((), generator=g).item()
        cx = r + (SIZE - 2 * r) * torch.rand((), generator=g).item()
        cy = r + (SIZE - 2 * r) * torch.rand((), generator=g).item()
        k = int(torch.randint(0, CLASSES, (), generator=g))
        dx, dy = xs - cx, ys - cy
        if k == 0:
            inside = dx * dx + dy * dy <= r * r
        elif k == 1:
            inside = (dx.abs() <= r) & (dy.abs() <= r)
        else:
            inside = (dy <= r) & (dy >= -r) & (dx.abs() <= (dy + r) / 2)
        if (mask[inside] > 0).any():
            continue                                            # keep the shapes apart
        img = torch.where(inside, 0.6 + 0.1 * k + 0.0 * img, img)
        mask[inside] = k + 1
        yy, xx = inside.nonzero(as_tuple=True)
        boxes.append([float(xx.min()), float(yy.min()), float(xx.max()) + 1, float(yy.max()) + 1])
        labels.append(k)
    img = (img + 0.05 * torch.randn(SIZE, SIZE, generator=g)).clamp(0, 1)
    return img[None], torch.tensor(boxes).reshape(-1, 4), torch.tensor(labels, dtype=torch.long), mask


def dataset(count: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    rows = [scene(g) for _ in range(count)]
    rows = [r for r in rows if len(r[2])]
    return (torch.stack([r[0] for r in rows]), [GroundTruth(r[1], r[2]) for r in rows], torch.stack([r[3] for r in rows]))


def main(steps: int = 300, device: str = "cpu", quiet: bool = False) -> dict:
    torch.manual_seed(0)
    x, truths, masks = dataset(600, 1)
    xt, truths_t, masks_t = dataset(100, 2)
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    g = torch.Generator().manual_seed(3)
    detector = CenterDetector(CLASSES, channels=1, width=16).to(device, dtype)
    segmenter = Segmenter(CLASSES + 1, channels=1, width=8).to(device, dtype)
    opt_d = torch.optim.AdamW(detector.parameters(), lr=2e-3)
    opt_s = torch.optim.AdamW(segmenter.parameters(), lr=3e-3)
    for step in range(steps):
        idx = torch.randint(0, len(x), (32,), generator=g).tolist()
        xb = x[idx].to(device, dtype)
        loss_d = detector.loss(detector(xb), [truths[i] for i in idx], SIZE, SIZE)
        opt_d.zero_grad()
        loss_d.backward()
        opt_d.step()
        loss_s = segmenter.loss(segmenter(xb), masks[idx].to(device))
        opt_s.zero_grad()
        loss_s.backward()
        opt_s.step()
        if not quiet and (step + 1) % 50 == 0:
            print(f"step {step + 1:4d}  detector {float(loss_d.detach()):.3f}  segmenter {float(loss_s.detach()):.3f}")
    detector.eval()
    segmenter.eval()
    found = detector.detect(xt.to(device, dtype), threshold=0.25)
    summary = mean_average_precision(found, truths_t)
    with torch.no_grad():
        predicted = segmenter(xt.to(device, dtype)).float().argmax(1).cpu()
    miou, per_class = mean_iou(predicted, masks_t, CLASSES + 1)
    if not quiet:
        print(f"detector: mAP@[.5:.95] {summary['map']:.3f}, mAP@.5 {summary['map50']:.3f}")
        print(f"segmenter: mean IoU {miou:.3f} per class {[round(v, 3) for v in per_class]}")
    return {"map": summary["map"], "map50": summary["map50"], "miou": miou}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=300)
    a = ap.parse_args()
    main(a.steps, a.device)
