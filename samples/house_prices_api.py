"""Tabular regression end to end: train a small network on synthetic house prices with scaled inputs, host it in the
inference engine as a predictor, and query it over HTTP (`POST /predict/houses`, `/predict/houses/batch`).

    python samples/house_prices_api.py                 # trains, then answers two requests through a test client
    python samples/house_prices_api.py --serve 8080    # trains, then serves until interrupted

Reference: samples/Idrak.Samples.HousePrices and HousePricesApi (Program.cs of each).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402
from idrak_b200.serve.api import create_app  # noqa: E402
from idrak_b200.serve.inference_engine import InferenceEngine  # noqa: E402
from idrak_b200.training.trainer import Trainer  # noqa: E402


def make_data(n: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    area = 40 + 160 * torch.rand(n, generator=g)              # square metres
    rooms = torch.randint(1, 7, (n,), generator=g).float()
    age = 60 * torch.rand(n, generator=g)                      # years
    price = 50 + 2.1 * area + 9.0 * rooms - 0.8 * age + 4.0 * torch.randn(n, generator=g)   # thousands
    return torch.stack([area, rooms, age], 1), price[:, None]


class Scaled(torch.nn.Module):
    """The network between an input scaler and an output scaler (what the reference's Predictor carries as scalers)."""

    def __init__(self, net, x_mean, x_std, y_mean, y_std):
        super().__init__()
        self.net = net
        for k, v in (("x_mean", x_mean), ("x_std", x_std), ("y_mean", y_mean), ("y_std", y_std)):
            self.register_buffer(k, v)

    def forward(self, x):
        single = x.dim() == 1
        x = x[None] if single else x
        y = self.net((x - self.x_mean) / self.x_std) * self.y_std + self.y_mean
        return y[0] if single else y


def train(epochs: int = 60):
    torch.manual_seed(0)
    x, y = make_data(2048)
    xm, xs, ym, ys = x.mean(0), x.std(0), y.mean(0), y.std(0)
    net = Network.input(3).linear(32).relu().linear(32).relu().linear(1).build()
    batches = [((x[i: i + 256] - xm) / xs, (y[i: i + 256] - ym) / ys) for i in range(0, 2048, 256)]
    Trainer(net, torch.optim.Adam(net.parameters(), lr=1e-2), torch.nn.functional.mse_loss).fit(batches, epochs=epochs)
    model = Scaled(net, xm, xs, ym, ys).eval()
    tx, ty = make_data(512, seed=1)
    with torch.no_grad():
        mae = float((model(tx) - ty).abs().mean())
    return model, mae


def main(argv=None) -> dict:
    argv = sys.argv[1:] if argv is None else argv
    model, mae = train()
    engine = InferenceEngine.create().add_predictor("houses", lambda: model).build()
    app = create_app(engine)
    if argv[:1] == ["--serve"]:
        import uvicorn
        uvicorn.run(app, host="127.0.0.1", port=int(argv[1]) if len(argv) > 1 else 8080)
        return {}
    from fastapi.testclient import TestClient
    with TestClient(app) as client:
        one = client.post("/predict/houses", json={"input": [120.0, 4, 10.0]}).json()
        many = client.post("/predict/houses/batch", json={"inputs": [[60.0, 2, 40.0], [180.0, 6, 1.0]]}).json()
    print(f"held-out mean absolute error {mae:.2f} thousand")
    print("120 m2, 4 rooms, 10 years ->", round(one["output"][0], 1))
    print("batch ->", [round(o[0], 1) for o in many["outputs"]])
    engine.close()
    return {"mae": mae, "one": one, "many": many}


if __name__ == "__main__":
    main()
