"""Pretrainer on CPU: the draw order is a function of (seed, stage, step) only, a staged run lowers the loss and
writes Hugging Face checkpoints, and a run resumed from a checkpoint - also on another number of ranks - continues
exactly where the first would have been."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from idrak_b200.formats.tokens import TokenFile, write_tokens
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.models.pretrained import load_pretrained
from idrak_b200.text.pretraining import (PretrainOptions, PretrainStage, Pretrainer, draw_global_batch, lr_at)

HERE = os.path.dirname(os.path.abspath(__file__))


def _tokens(path, n=6000, vocab=300, seed=0):
    rng = np.random.default_rng(seed)
    base = rng.integers(0, vocab, size=40)
    ids = np.concatenate([np.roll(base, int(rng.integers(0, 5))) for _ in range(n // 40)])   # learnable structure
    write_tokens(path, ids, vocab)
    return str(path)


def _model():
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=300, max_positions=64)
    return build_decoder(spec, seed=3).float()


def test_draw_order_and_schedule(tmp_path):
    a, b = _tokens(tmp_path / "a.tokens"), _tokens(tmp_path / "b.tokens", n=2000, seed=1)
    files = [TokenFile(a, 32), TokenFile(b, 32)]
    d1 = draw_global_batch(files, None, 5, 0, 7, 16)
    assert d1 == draw_global_batch(files, None, 5, 0, 7, 16) != draw_global_batch(files, None, 5, 0, 8, 16)
    assert all(0 <= w < len(files[f]) for f, w in d1)
    only_b = draw_global_batch(files, [0.0, 1.0], 5, 1, 0, 16)
    assert {f for f, _ in only_b} == {1}
    o = PretrainOptions(learning_rate=1.0, warmup_steps=10, min_lr_ratio=0.1)
    assert lr_at(0, 100, o) == pytest.approx(0.1) and lr_at(9, 100, o) == pytest.approx(1.0)
    assert lr_at(100, 100, o) == pytest.approx(0.1) and 0.5 < lr_at(50, 100, o) < 0.65


def test_staged_run_checkpoints_and_exact_resume(tmp_path):
    a, b = _tokens(tmp_path / "a.tokens"), _tokens(tmp_path / "b.tokens", seed=1)
    stages = [PretrainStage("one", [a], steps=6, seq_len=32), PretrainStage("two", [a, b], steps=6, seq_len=32, weights=[1, 3])]
    o = PretrainOptions(stages=stages, global_batch=8, micro_batch=4, learning_rate=3e-3, warmup_steps=2, save_every=4,
                        out_dir=str(tmp_path / "run"), eval_files=[a], eval_every=6, eval_batches=2, seed=11)
    seen = []
    res = Pretrainer.train(_model(), o, progress=lambda s, l: seen.append(s))
    assert res.steps == 12 and res.losses[-1] < res.losses[0] - 0.3 and res.tokens == 12 * 8 * 32
    assert len(res.eval_losses) == 2 and seen[-1] == 12
    ck = tmp_path / "run" / "checkpoint-4"
    st = json.loads((ck / "train-state.json").read_text())
    assert st["step"] == 4 and st["stage"] == 0 and st["world"] == 1
    assert (ck / "optimizer.safetensors").exists() and (ck / "config.json").exists()
    reloaded = load_pretrained(str(tmp_path / "run" / "checkpoint-12"))
    assert reloaded.spec.dim == 64
    # resume from step 4: the remaining eight losses repeat
    o2 = PretrainOptions(**{**o.__dict__, "resume_from": str(ck), "out_dir": None, "save_every": 0, "eval_every": 0})
    res2 = Pretrainer.train(_model(), o2)
    assert res2.steps == 12 and np.allclose(res2.losses, res.losses[4:], rtol=2e-4, atol=2e-4)
    with pytest.raises(ValueError, match="another global batch or seed"):
        Pretrainer.train(_model(), PretrainOptions(**{**o2.__dict__, "seed": 12}))


def _ranks(nproc, tokens, out, steps, resume, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "pretrain_worker.py"), tokens, str(out), str(steps),
           resume]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return json.loads((out / "losses.json").read_text())


def test_same_data_on_any_world_size_and_resume_across_world_sizes(tmp_path):
    tokens = _tokens(tmp_path / "a.tokens")
    (tmp_path / "w1").mkdir(); (tmp_path / "w2").mkdir(); (tmp_path / "w2r").mkdir()
    one = _ranks(1, tokens, tmp_path / "w1", 6, "-", 29671)
    two = _ranks(2, tokens, tmp_path / "w2", 6, "-", 29672)
    assert np.allclose(one, two, rtol=1e-3, atol=1e-3)               # same global batches, same losses
    # first three steps on one rank, the rest on two
    (tmp_path / "w1s").mkdir()
    _ranks(1, tokens, tmp_path / "w1s", 3, "-", 29673)
    rest = _ranks(2, tokens, tmp_path / "w2r", 6, str(tmp_path / "w1s" / "checkpoint-3"), 29674)
    assert np.allclose(rest, one[3:], rtol=1e-3, atol=1e-3)
