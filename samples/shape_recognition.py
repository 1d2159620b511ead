"""Image classification with a convolutional network: 16 x 16 grayscale drawings of circles, squares, triangles and
crosses at random positions and sizes, with noise. Conv2d, BatchNorm, MaxPool2d and Dropout through the network builder;
on a GPU in bf16 the convolutions run as patch rows around the tensor-core GEMM and the pools on the package's kernels.

    python samples/shape_recognition.py [--device cuda]

Reference: samples/Idrak.Samples.ShapeRecognition/Program.cs.
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402

SHAPES = ("circle", "square", "triangle", "cross")


def draw(shape: str, g: torch.Generator, size: int = 16) -> torch.Tensor:
    """One drawing: the outline of ``shape`` at a random place and size, values in [0, 1], plus noise."""
    r = 3.0 + 3.0 * torch.rand((), generator=g).item()
    cx = r + 1 + (size - 2 * r - 2) * torch.rand((), generator=g).item()
    cy = r + 1 + (size - 2 * r - 2) * torch.rand((), generator=g).item()
    ys, xs = torch.meshgrid(torch.arange(size).float(), torch.arange(size).float(), indexing="ij")
    dx, dy = xs - cx, ys - cy
    if shape == "circle":
        d = (torch.sqrt(dx * dx + dy * dy) - r).abs()
    elif shape == "square":
        d = (torch.maximum(dx.abs(), dy.abs()) - r).abs()
    elif shape == "cross":
        d = torch.minimum(dx.abs() + (dy.abs() > r) * 99, dy.abs() + (dx.abs() > r) * 99)
    else:                                                        # triangle: three edges of an upright one
        h = r * math.sqrt(3) / 2
        base = (dy - h * 0.6).abs() + (dx.abs() > r) * 99
        left = ((dy + h * 1.4) * (r / (2 * h)) + dx).abs() * 0.9 + ((dy < -h * 1.4) | (dy > h * 0.6)) * 99
        right = ((dy + h * 1.4) * (r / (2 * h)) - dx).abs() * 0.9 + ((dy < -h * 1.4) | (dy > h * 0.6)) * 99
        d = torch.minimum(base, torch.minimum(left, right))
    img = (1.0 - d).clamp(0, 1)
    return (img + 0.1 * torch.randn(size, size, generator=g)).clamp(0, 1)


def dataset(count: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, len(SHAPES), (count,), generator=g)
    images = torch.stack([draw(SHAPES[int(k)], g) for k in labels])[:, None]
    return images, labels


def augment(x: torch.Tensor, g: torch.Generator) -> torch.Tensor:
    """Flip left-right, shift by up to one pixel, add noise: differently each epoch."""
    flip = torch.rand(len(x), generator=g) < 0.5
    x = torch.where(flip[:, None, None, None], x.flip(-1), x)
    sx, sy = (int(v) for v in torch.randint(-1, 2, (2,), generator=g))
    x = torch.roll(x, (sy, sx), (-2, -1))
    return (x + 0.05 * torch.randn(x.shape, generator=g)).clamp(0, 1)


def build():
    return (Network.image(1, 16, 16).conv2d(16, 3, padding=1).batch_norm().relu().max_pool2d(2)
            .conv2d(32, 3, padding=1).batch_norm().relu().max_pool2d(2).flatten().dropout(0.2)
            .linear(64).relu().linear(len(SHAPES)).build())


def main(epochs: int = 12, device: str = "cpu", quiet: bool = False) -> dict:
    torch.manual_seed(0)
    x, y = dataset(1600, 1)
    xt, yt = dataset(400, 2)
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    model = build().to(device, dtype)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3 if dtype == torch.float32 else 2e-3)
    g = torch.Generator().manual_seed(3)
    for epoch in range(epochs):
        model.train()
        order = torch.randperm(len(x), generator=g)
        total = 0.0
        for i in range(0, len(x), 100):
            idx = order[i:i + 100]
            xb = augment(x[idx], g).to(device, dtype)
            loss = torch.nn.functional.cross_entropy(model(xb).float(), y[idx].to(device))
            opt.zero_grad()
            loss.backward()
            opt.step()
            total += float(loss.detach())
        if not quiet:
            print(f"epoch {epoch + 1:2d}  loss {total / (len(x) // 100):.4f}")
    model.eval()
    with torch.no_grad():
        pred = model(xt.to(device, dtype)).float().argmax(-1).cpu()
    accuracy = float((pred == yt).float().mean())
    if not quiet:
        print(f"held-out accuracy {accuracy:.3f}")
        for k, name in enumerate(SHAPES):
            row = [int(((pred == j) & (yt == k)).sum()) for j in range(len(SHAPES))]
            print(f"{name:9s} -> {row}")
    return {"accuracy": accuracy, "model": model}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--epochs", type=int, default=12)
    a = ap.parse_args()
    main(a.epochs, a.device)
