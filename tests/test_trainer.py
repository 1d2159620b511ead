"""Trainer: fit / evaluate, callbacks, schedules, early stopping, stop file + bit-exact resume (CPU)."""
import json
import math
import os

import pytest
import torch

from idrak_b200.diag import Level, MetricsRecorder, Telemetry
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.ops import FusedAdamW, FusedSGD
from idrak_b200.training import (CsvLogger, EarlyStopping, Metrics, Trainer, TrainerCallback, WarmupCosine, Cosine,
                                 StepDecay)


def _xor_data():
    x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]]).repeat(16, 1)
    y = (x[:, :1] != x[:, 1:]).float()
    return [(x[i:i + 16], y[i:i + 16]) for i in range(0, 64, 16)]


def _mlp(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(2, 16), torch.nn.Tanh(), torch.nn.Linear(16, 1), torch.nn.Sigmoid())


def test_fit_learns_xor_with_metrics_callbacks_and_telemetry(tmp_path):
    model = _mlp()
    opt = FusedAdamW(model.parameters(), lr=5e-2, weight_decay=0.0)
    seen = []

    class Spy(TrainerCallback):
        def on_train_begin(self, t): seen.append("begin")
        def on_batch_end(self, t, e): seen.append("batch")
        def on_epoch_end(self, t, e): seen.append("epoch")
        def on_train_end(self, t, h): seen.append("end")

    rec = Telemetry.add(MetricsRecorder())
    try:
        tr = Trainer(model, opt, torch.nn.functional.binary_cross_entropy, metrics=[Metrics.accuracy],
                     callbacks=[Spy(), CsvLogger(tmp_path / "log.csv")])
        hist = tr.fit(_xor_data(), epochs=60, validation=_xor_data())
    finally:
        Telemetry.remove(rec)
    assert hist.epochs[-1].loss < 0.2 and hist.epochs[-1].metrics["accuracy"] > 0.95
    assert hist.epochs[-1].validation_loss is not None
    assert seen[0] == "begin" and seen[-1] == "end" and seen.count("epoch") == 60 and seen.count("batch") == 240
    assert len(rec.series["EpochCompleted.loss"]) == 60 and len(rec.series["BatchCompleted.loss"]) == 240
    assert (tmp_path / "log.csv").read_text().count("\n") == 61
    assert not Telemetry.is_enabled(Level.BATCHES)
    res = tr.evaluate(_xor_data())
    assert res.samples == 64 and res.metrics["accuracy"] > 0.95
    assert tr.predict(torch.tensor([[0., 1.]])).item() > 0.5


def test_early_stopping_restores_best_weights():
    model = _mlp(1)
    opt = FusedSGD(model.parameters(), lr=0.5, momentum=0.9)
    tr = Trainer(model, opt, torch.nn.functional.mse_loss, early_stopping_patience=2)
    flipped = [(x, 1.0 - y) for x, y in _xor_data()]      # validation gets worse as training gets better
    hist = tr.fit(_xor_data(), epochs=50, validation=flipped)
    assert hist.stopped_early and len(hist.epochs) < 50
    best = hist.epochs[hist.best_epoch].validation_loss
    assert abs(tr.evaluate(flipped).loss - best) < 1e-6


def test_schedules():
    s = WarmupCosine(1.0, warmup=10, total=110, min_lr=0.1)
    assert s.lr(0) == pytest.approx(0.1) and s.lr(9) == pytest.approx(1.0)
    assert s.lr(60) == pytest.approx(0.55) and s.lr(110) == pytest.approx(0.1) and s.lr(500) == pytest.approx(0.1)
    assert Cosine(2.0, 100).lr(50) == pytest.approx(1.0)
    assert StepDecay(1.0, 10, 0.5).lr(25) == pytest.approx(0.25)
    opt = FusedAdamW(_mlp().parameters(), lr=1.0)
    s.apply(opt, 4)
    assert opt.lr == pytest.approx(0.5)


def _lm_batches(seed, n=6):
    g = torch.Generator().manual_seed(seed)
    data = torch.randint(0, 256, (n, 4, 33), generator=g)
    return [(d[:, :-1], d[:, 1:]) for d in data]


def _lm_trainer(folder=None, resume=None, stop=None):
    spec = DecoderSpec.gpt2(layers=1, dim=32, heads=2, vocab=256, max_positions=32)
    model = build_decoder(spec, seed=3)
    opt = FusedAdamW(model.decay_groups(0.1), lr=1e-2, max_grad_norm=1.0)
    return Trainer(model, opt, None, checkpoint_folder=folder, resume_from=resume, stop_folder=stop,
                   scheduler=WarmupCosine(1e-2, 2, 20))


def test_stop_file_checkpoint_and_resume_is_bit_exact(tmp_path):
    # uninterrupted run
    full = _lm_trainer()
    full.fit(_lm_batches(0), epochs=2)
    ref = torch.cat([p.detach().reshape(-1) for p in full.model.parameters()])

    # interrupted after 4 steps of the first epoch by a stop file
    ck = tmp_path / "ck"
    ck.mkdir()

    class StopAt(TrainerCallback):
        def on_batch_end(self, t, e):
            if e.step == 3:
                (ck / "stop").write_text("")

    a = _lm_trainer(folder=str(ck), stop=str(ck))
    a.callbacks.append(StopAt())
    hist = a.fit(_lm_batches(0), epochs=2)
    assert hist.stopped_by_request and a.global_step == 4
    state = json.loads((ck / "checkpoint-4" / "train-state.json").read_text())
    assert state["epoch"] == 0 and state["step_in_epoch"] == 4
    # the reference's keys (Trainer.cs WriteState): format, step, best_epoch, since_best, dropout_draws
    assert state["format"] == "idrak-train-state/2" and state["step"] == 4
    assert {"best_epoch", "since_best", "dropout_draws"} <= set(state)
    assert {p.name for p in (ck / "checkpoint-4").iterdir()} == {"model.ikw", "optimizer.safetensors", "train-state.json",
                                                                 "rng-state.pt"}
    os.remove(ck / "stop")

    b = _lm_trainer(resume=str(ck))
    b.fit(_lm_batches(0), epochs=2)
    got = torch.cat([p.detach().reshape(-1) for p in b.model.parameters()])
    assert b.global_step == 12 and torch.equal(got, ref)


def test_checkpoint_keep_and_optimizer_state_names(tmp_path):
    t = _lm_trainer(folder=str(tmp_path))
    t.checkpoint_keep = 2
    t.fit(_lm_batches(1, n=2), epochs=4)
    kept = sorted(p.name for p in tmp_path.iterdir() if p.is_dir())
    assert kept == ["checkpoint-6", "checkpoint-8"]
    from idrak_b200.formats.safetensors import SafeTensorsReader
    with SafeTensorsReader.open(tmp_path / "checkpoint-8" / "optimizer.safetensors") as r:
        names = set(r.keys())
        assert "step" in names and "m.0" in names and "v.0" in names
        assert r.metadata["format"] == "idrak-optimizer"
        assert float(r.read("step")) == 8.0


def test_training_run_is_the_trainer_as_one_object():
    import dataclasses
    from idrak_b200.training import TrainingRun
    run = TrainingRun(model=_mlp(), loss=torch.nn.functional.binary_cross_entropy,
                      optimizer=lambda p: FusedAdamW(p, lr=5e-2, weight_decay=0.0), train=_xor_data(), epochs=30,
                      validation=_xor_data(), metrics=[Metrics.accuracy], max_gradient_norm=1.0)
    history = run.fit()
    assert run.trainer is not None and history.epochs[-1].metrics["accuracy"] == 1.0
    variant = dataclasses.replace(run, model=_mlp(1), epochs=2, max_gradient_norm=0.5)
    assert variant.epochs == 2 and run.epochs == 30
    assert len(variant.fit().epochs) == 2 and variant.trainer.max_gradient_norm == 0.5


def test_resume_from_a_reference_style_checkpoint_folder(tmp_path):
    """A folder laid out the way the reference's trainer writes it: train-state.json with format / step / best_loss /
    best_epoch / since_best / dropout_draws only, model.ikw, optimizer.safetensors, best-weights.safetensors with one
    flat entry per tensor named by position. The step count places the resume inside the epoch."""
    from idrak_b200.formats import ikw
    from idrak_b200.formats.safetensors import save_file
    src = _lm_trainer()
    src.fit(_lm_batches(0), epochs=1)
    ck = tmp_path / "checkpoint-6"
    ck.mkdir()
    ikw.save_module(src.model, ck / "model.ikw")
    save_file({k: v.float().contiguous() for k, v in src.optimizer.state_dict().items()}, ck / "optimizer.safetensors",
              metadata={"format": "idrak-optimizer", "optimizer": "AdamW"})
    best = {str(i): torch.full((v.numel(),), float(i)) for i, v in enumerate(src.model.state_dict().values())}
    save_file(best, ck / "best-weights.safetensors", metadata={"format": "idrak-best-weights"})
    (ck / "train-state.json").write_text(json.dumps(
        {"format": "idrak-train-state/2", "step": 6, "best_epoch": 0, "since_best": 1, "dropout_draws": [],
         "best_loss": 1.25}) + "\n")
    t = _lm_trainer(resume=str(ck))
    state = t.load_checkpoint(ck)
    assert t.global_step == 6 and state["best_loss"] == 1.25 and state["since_best"] == 1
    first = next(iter(state["_best_weights"].values()))
    assert float(first.float().mean()) == 0.0 and len(state["_best_weights"]) == len(best)
    hist = t.fit(_lm_batches(0), epochs=2)          # 6 steps per epoch: resumes at the start of the second epoch
    assert t.global_step == 12 and len(hist.epochs) == 1 and hist.epochs[0].epoch == 1

    bad = tmp_path / "checkpoint-7"
    bad.mkdir()
    (bad / "train-state.json").write_text(json.dumps({"format": "idrak-train-state/2", "best_epoch": 0}))
    ikw.save_module(src.model, bad / "model.ikw")
    with pytest.raises(ValueError, match="names no step"):
        _lm_trainer().load_checkpoint(bad)


def test_early_stopping_state_survives_a_checkpoint(tmp_path):
    t = _lm_trainer(folder=str(tmp_path))
    t.early_stopping_patience, t.restore_best_weights = 50, True
    t.fit(_lm_batches(2, n=2), epochs=3)
    newest = sorted(tmp_path.glob("checkpoint-*"), key=lambda p: int(p.name.split("-")[1]))[-1]
    state = json.loads((newest / "train-state.json").read_text())
    assert "best_loss" in state and state["best_epoch"] >= 0 and (newest / "best-weights.safetensors").exists()
    r = _lm_trainer(resume=str(newest))
    loaded = r.load_checkpoint(newest)
    assert loaded["best_loss"] == state["best_loss"] and "_best_weights" in loaded
