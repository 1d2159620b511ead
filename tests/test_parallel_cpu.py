"""Pipeline parallelism, local SGD and gradient compression on gloo CPU ranks."""
import json
import os
import subprocess
import sys

import pytest
import torch

from idrak_b200.parallel.pipeline import ideal_bubble, in_flight, schedule_order, split_layers

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
_PORT = [29680]


def _ranks(nproc, *args):
    _PORT[0] += 1
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(_PORT[0]), os.path.join(HERE, "parallel_worker.py"), *[str(a) for a in args]]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]


def test_schedules_and_layer_split():
    assert schedule_order("gpipe", 0, 3, 2) == [("F", 0), ("F", 1), ("B", 1), ("B", 0)]
    o = schedule_order("1f1b", 0, 3, 4)
    assert o[:3] == [("F", 0), ("F", 1), ("F", 2)] and o[3:5] == [("B", 0), ("F", 3)]
    for name in ("gpipe", "1f1b"):
        for s in range(3):
            order = schedule_order(name, s, 3, 5)
            assert sorted(m for k, m in order if k == "F") == list(range(5)) == sorted(m for k, m in order if k == "B")
            for m in range(5):
                assert order.index(("F", m)) < order.index(("B", m))
    assert in_flight("gpipe", 0, 4, 8) == 8 and in_flight("1f1b", 0, 4, 8) == 4 and in_flight("1f1b", 3, 4, 8) == 1
    assert ideal_bubble(4, 12) == pytest.approx(3 / 15)
    assert split_layers(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        split_layers(2, 3)
    with pytest.raises(KeyError, match="not registered"):
        schedule_order("zigzag", 0, 2, 2)


def _single(tie, steps=3):
    from parallel_worker import _data, _model
    from idrak_b200.ops import FusedAdamW
    model = _model(tie)
    opt = FusedAdamW(model.decay_groups(0.1), lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    data = _data(steps)
    losses = []
    for s in range(steps):
        b = data[s]
        opt.zero_grad()
        loss = model.loss(b[:, :-1].int(), b[:, 1:].int())
        loss.backward()
        opt.step()
        losses.append(float(loss))
    return losses, model


@pytest.mark.parametrize("stages,schedule,tie,nproc", [(2, "gpipe", "tie", 2), (4, "1f1b", "untied", 4)])
def test_pipeline_matches_single_process(stages, schedule, tie, nproc, tmp_path):
    out = tmp_path / "p.pt"
    _ranks(nproc, "pipeline", out, stages, schedule, tie)
    got = torch.load(out)
    losses, model = _single(tie == "tie")
    assert max(abs(a - b) for a, b in zip(got["losses"], losses)) < 2e-4
    ref = dict(model.named_parameters())
    from idrak_b200.parallel.pipeline import split_layers as sl
    ranges = sl(4, stages)
    checked = 0
    for stage, replica, state in got["states"]:
        lo, _ = ranges[stage]
        for name, t in state.items():
            n = name.split(".", 2)[2]
            if n.startswith("blocks."):
                i, rest = n.split(".", 2)[1:]
                n = f"blocks.{int(i) + lo}.{rest}"
            assert (t - ref[n].detach()).abs().max().item() < 2e-4, name
            checked += 1
    assert checked >= len(ref)


def test_pipeline_with_replicas(tmp_path):
    out = tmp_path / "p.pt"
    _ranks(4, "pipeline", out, 2, "gpipe", "untied")
    got = torch.load(out)
    # both replicas of a stage end with identical weights
    by_stage = {}
    for stage, replica, state in got["states"]:
        by_stage.setdefault(stage, []).append(state)
    for stage, copies in by_stage.items():
        assert len(copies) == 2
        for k in copies[0]:
            assert torch.equal(copies[0][k], copies[1][k])
    assert got["losses"][2] < got["losses"][0]


@pytest.mark.parametrize("momentum", [0.0, 0.9])
def test_local_sgd_averages_every_k_steps(momentum, tmp_path):
    out = tmp_path / "l.json"
    _ranks(2, "localsgd", out, 4, momentum)
    r = json.loads(out.read_text())
    assert r["syncs"] == 2 and [s for s, _ in r["spread"]] == [False, False, False, True] * 2
    assert all(d > 0 for s, d in r["spread"] if not s) and all(d < 1e-6 for s, d in r["spread"] if s)


@pytest.mark.parametrize("kind,ratio,error", [("none", 1.0, 1e-5), ("bf16", 0.5, 0.1), ("int8", 0.33, 0.05),
                                              ("fp8", 0.33, 0.3), ("top-k", 0.21, 4.0)])
def test_gradient_compression_kinds(kind, ratio, error, tmp_path):
    out = tmp_path / "c.json"
    _ranks(2, "compress", out, kind)
    r = json.loads(out.read_text())
    assert r["identical_on_ranks"] and r["ratio"] <= ratio + 0.01
    # with error feedback what was left out arrives later: the running sums stay close to the true ones
    assert r["accumulated_error"] < error, r
    from idrak_b200.parallel.compression import Compressor
    with pytest.raises(KeyError, match="not registered"):
        Compressor("zip")


def test_fused_dp_bucket_count_is_bounded_by_the_flag_channels():
    """Bucket b signals on flag channel CH_BUCKET0 + b and the one after it; a layout with more buckets than the flag
    area has rows must be refused (the layout code then doubles the bucket size until it fits)."""
    from idrak_b200.parallel.comm import CH_BUCKET0
    from idrak_b200.parallel.dp import bucket_channels_fit
    channels = 512
    assert bucket_channels_fit(1, channels)
    assert bucket_channels_fit(channels - CH_BUCKET0 - 1, channels)
    assert not bucket_channels_fit(channels - CH_BUCKET0, channels)
    assert not bucket_channels_fit(10_000, channels)
