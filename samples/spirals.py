"""Two interleaved spirals: a small classifier built with the network builder, trained with early stopping on a held-out
split, and its decision boundary sampled on a grid.

    python samples/spirals.py

Reference: samples/Idrak.Samples.Spirals/Program.cs.
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402
from idrak_b200.training.trainer import Trainer  # noqa: E402


def spirals(points: int, noise: float, seed: int):
    g = torch.Generator().manual_seed(seed)
    t = torch.rand(points, generator=g) * 3.0 * math.pi + 0.5
    label = torch.randint(0, 2, (points,), generator=g)
    angle = t + label * math.pi
    xy = torch.stack([t * torch.cos(angle), t * torch.sin(angle)], 1) / 10.0
    return xy + torch.randn(points, 2, generator=g) * noise, label


def main(epochs: int = 150, quiet: bool = False) -> dict:
    torch.manual_seed(0)
    x, y = spirals(1200, 0.01, 1)
    xt, yt = spirals(400, 0.01, 2)
    model = Network.input(2).linear(64).tanh().linear(64).tanh().linear(2).build()
    trainer = Trainer(model, torch.optim.Adam(model.parameters(), lr=1e-2), torch.nn.functional.cross_entropy,
                      early_stopping_patience=40)
    batches = [(x[i:i + 200], y[i:i + 200]) for i in range(0, len(x), 200)]
    trainer.fit(batches, epochs=epochs, validation=[(xt, yt)])
    accuracy = float((trainer.predict(xt).argmax(-1) == yt).float().mean())
    side = torch.linspace(-1.1, 1.1, 24)
    grid = torch.stack(torch.meshgrid(side, side, indexing="xy"), -1).reshape(-1, 2)
    picture = trainer.predict(grid).argmax(-1).reshape(24, 24)
    if not quiet:
        print(f"held-out accuracy {accuracy:.3f}")
        for row in picture.flip(0).tolist():
            print("".join("#" if v else "." for v in row))
    return {"accuracy": accuracy, "picture": picture}


if __name__ == "__main__":
    main()
