"""ONNX round trip without the onnx package: a small image classifier is exported to an ONNX file, the file is loaded
back as a module, both give the same outputs, and the loaded module is fine-tuned further.

    python samples/onnx_import.py

Reference: samples/Idrak.Samples.OnnxImport/Program.cs.
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402
from idrak_b200 import onnx  # noqa: E402


def main(quiet: bool = False) -> dict:
    torch.manual_seed(0)
    model = (Network.image(1, 12, 12).conv2d(4, 3, padding=1).relu().max_pool2d(2).flatten().linear(16).relu()
             .linear(3).build())
    x = torch.randn(5, 1, 12, 12)
    data = onnx.export(model, ["N", 1, 12, 12])
    with tempfile.TemporaryDirectory() as folder:
        path = os.path.join(folder, "classifier.onnx")
        with open(path, "wb") as f:
            f.write(data)
        loaded = onnx.load(path, trainable=True)
    same = float((loaded(x) - model(x)).detach().abs().max())
    # the imported graph trains: its initialisers are parameters
    target = torch.tensor([0, 1, 2, 1, 0])
    opt = torch.optim.Adam(loaded.parameters(), lr=0.05)
    first = last = None
    for _ in range(40):
        loss = torch.nn.functional.cross_entropy(loaded(x), target)
        first = float(loss) if first is None else first
        opt.zero_grad()
        loss.backward()
        opt.step()
        last = float(loss)
    out = {"bytes": len(data), "largest_difference": same, "first_loss": first, "last_loss": last,
           "parameters": sum(p.numel() for p in loaded.parameters())}
    if not quiet:
        print(out)
    return out


if __name__ == "__main__":
    main()
