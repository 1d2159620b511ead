"""Parameter sharding against plain single-process training of the same model on the same global batches."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _reference(steps):
    from zero3_worker import make_data, make_model
    model = make_model()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.0)
    data = make_data(steps)
    losses = []
    for s in range(steps):
        b = data[s]
        loss = model.loss(b[:, :-1].contiguous(), b[:, 1:].contiguous())
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()))
    return losses, model.state_dict()


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_parameters_train_like_the_whole_model(tmp_path, world):
    out = tmp_path / "out.pt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29790 + world), os.path.join(HERE, "zero3_worker.py"), str(out), "4"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = torch.load(out)
    losses, state = _reference(4)
    assert got["losses"] == pytest.approx(losses, abs=2e-4)
    for k, v in state.items():
        assert torch.allclose(got["state"][k], v, atol=2e-4), k
    if world == 2:
        assert got["held"] < 0.75 * got["total"]            # the blocks' weights are halved per rank
