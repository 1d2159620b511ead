"""XOR with a two-layer network described through the network builder, trained by `Trainer`, then described as JSON
and rebuilt from it.

    python samples/xor.py

Reference: samples/Idrak.Samples.Xor/Program.cs.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402
from idrak_b200.training.trainer import Trainer  # noqa: E402


def main(epochs: int = 600, quiet: bool = False) -> dict:
    torch.manual_seed(0)
    x = torch.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
    y = torch.tensor([[0.0], [1.0], [1.0], [0.0]])
    builder = Network.input(2).linear(8).tanh().linear(1).sigmoid()
    model = builder.build()
    trainer = Trainer(model, torch.optim.Adam(model.parameters(), lr=0.05), torch.nn.functional.binary_cross_entropy)
    history = trainer.fit([(x, y)], epochs=epochs)
    out = trainer.predict(x)
    description = builder.to_json()
    again = Network.from_json(description).build()
    again.load_state_dict(model.state_dict())
    same = torch.allclose(again(x), model(x))
    if not quiet:
        for row, p in zip(x.tolist(), out.flatten().tolist()):
            print(f"{int(row[0])} xor {int(row[1])} -> {p:.3f}")
        print("rebuilt from its description:", same)
    return {"predictions": out.flatten().tolist(), "rebuilt_matches": same, "epochs": len(history.epochs) if hasattr(history, "epochs") else epochs}


if __name__ == "__main__":
    main()
