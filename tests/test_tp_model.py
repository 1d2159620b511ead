"""A decoder sliced over tensor-parallel ranks trains like the unsliced one: on CPU with gloo ranks (collective
fallback path) and on GPUs with the fused kernels."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _run(device, mode, family, out, nproc, port, steps=3):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_model_worker.py"), device,
           mode, family, str(out), str(steps)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return torch.load(out)


def _single(family, device, dtype, steps=3):
    from tp_model_worker import make_data, make_spec
    from idrak_b200.models import build_decoder
    from idrak_b200.ops import FusedAdamW
    model = build_decoder(make_spec(family), seed=7).to(device, dtype)
    opt = FusedAdamW(model.decay_groups(0.1), lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    data = make_data(steps)
    losses = []
    for s in range(steps):
        b = data[s].to(device)
        opt.zero_grad()
        loss = model.loss(b[:, :-1].contiguous().int(), b[:, 1:].contiguous().int())
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
    return {"losses": losses, "embed": model.embed.detach().float().cpu(),
            "down0": model.blocks[0].mlp.down_weight.detach().float().cpu(), "norm": model.norm.weight.detach().float().cpu()}


@pytest.mark.parametrize("family", ["llama", "gpt2"])
def test_tp_decoder_matches_unsliced_on_cpu_ranks(family, tmp_path):
    got = _run("cpu", "nccl", family, tmp_path / "tp.pt", 2, 29661 if family == "llama" else 29662)
    ref = _single(family, "cpu", torch.float32)
    assert max(abs(a - b) for a, b in zip(got["losses"], ref["losses"])) < 2e-4
    for k in ("embed", "down0", "norm"):
        assert (got[k] - ref[k]).abs().max().item() < 2e-4, k


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["fused", "nccl"])
def test_tp_decoder_matches_unsliced_on_two_gpus(mode, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    got = _run("cuda", mode, "llama", tmp_path / "tp.pt", 2, 29663 if mode == "fused" else 29664)
    ref = _single("llama", "cuda", torch.bfloat16)
    assert max(abs(a - b) for a, b in zip(got["losses"], ref["losses"])) < 0.05
    for k in ("embed", "down0", "norm"):
        assert (got[k] - ref[k]).abs().max().item() < 2e-2, k
