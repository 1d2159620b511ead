"""``Trainer``: epochs over a batch source with metrics, callbacks, early stopping, learning-rate
schedule, gradient clipping, checkpoints with stop / resume, data-parallel sync and an out-of-memory
policy.

    trainer = Trainer(model, optimizer, loss)           # loss(predictions, targets) -> scalar tensor
    history = trainer.fit(train_batches, epochs=3, validation=val_batches)

A batch source is any iterable of ``(inputs, targets)`` (re-iterable per epoch). For language models
pass ``loss=None``: the model's own fused ``loss(inputs, targets)`` is used.

Checkpoints are folders ``checkpoint-STEP/`` holding ``model.ikw``, ``optimizer.safetensors`` (entries
``step``, ``m.{i}``, ``v.{i}``) and ``train-state.json``; ``resume_from`` restores them and redraws the
finished steps of the interrupted epoch without training so the data order continues where it stopped.
A file named ``stop`` appearing in ``stop_folder`` ends the run at the next step boundary with a
checkpoint (on several ranks the decision is agreed through the gradient sync's header).

Reference: Trainer (src/Idrak/Training/Trainer.cs:108,268-668), TrainerCallbacks.cs, TrainingRun.cs,
OutOfMemoryPolicies (src/Idrak.Abstraction/Training/OutOfMemoryPolicies.cs).
"""
from __future__ import annotations

import csv
import json
import math
import os
import shutil
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..diag.telemetry import BatchCompleted, EpochCompleted, Level, Telemetry
from ..formats import ikw
from ..formats.safetensors import SafeTensorsReader, save_file
from .schedules import Schedule


# --------------------------------------------------------------------------- metrics
@dataclass
class Metric:
    name: str
    batch_mean: Callable[[torch.Tensor, torch.Tensor], torch.Tensor]
    finalize: Optional[Callable[[float], float]] = None


def _match_rate(p, t, threshold=0.5):
    return ((p > threshold).float() == t.float()).float().mean()


class Metrics:
    mean_absolute_error = Metric("mae", lambda p, t: (p.float() - t.float()).abs().mean())
    mean_squared_error = Metric("mse", lambda p, t: (p.float() - t.float()).pow(2).mean())
    root_mean_squared_error = Metric("rmse", lambda p, t: (p.float() - t.float()).pow(2).mean(), math.sqrt)
    accuracy = Metric("accuracy", _match_rate)
    sparse_accuracy = Metric("accuracy", lambda p, t: (p.argmax(-1) == t.long()).float().mean())

    @staticmethod
    def binary_accuracy(threshold=0.5):
        return Metric("accuracy", lambda p, t: _match_rate(p, t, threshold))


@dataclass
class EvaluationResult:
    loss: float
    metrics: Dict[str, float]
    samples: int


@dataclass
class TrainingHistory:
    epochs: List[EpochCompleted] = field(default_factory=list)
    stopped_early: bool = False
    stopped_by_request: bool = False
    best_epoch: int = -1
    best_loss: float = math.inf


# --------------------------------------------------------------------------- callbacks
TRAIN_STATE_FORMAT = "idrak-train-state/2"


def _dropout_layers(model: torch.nn.Module):
    return [m for m in model.modules() if isinstance(m, (torch.nn.Dropout, torch.nn.Dropout1d, torch.nn.Dropout2d))
            or hasattr(m, "draws")]


def dropout_draws(model: torch.nn.Module) -> list:
    """How many masks each dropout layer has drawn (layers that count them expose ``draws``; PyTorch's own dropout
    draws from the global generator, whose state is checkpointed beside the json, and reports 0)."""
    return [int(getattr(m, "draws", 0)) for m in _dropout_layers(model)]


def restore_dropout_draws(model: torch.nn.Module, draws, where) -> None:
    layers = _dropout_layers(model)
    if len(draws) != len(layers):
        raise ValueError(f"{where} was written for a model with {len(draws)} dropout layers; this one has "
                         f"{len(layers)}: resume the run with its own model")
    for m, d in zip(layers, draws):
        if hasattr(m, "advance"):
            m.advance(max(0, int(d) - int(getattr(m, "draws", 0))))
        elif hasattr(m, "draws"):
            m.draws = int(d)


class TrainerCallback:
    def on_train_begin(self, trainer: "Trainer"): ...
    def on_batch_end(self, trainer: "Trainer", event: BatchCompleted): ...
    def on_epoch_end(self, trainer: "Trainer", event: EpochCompleted): ...
    def on_train_end(self, trainer: "Trainer", history: TrainingHistory): ...


class CsvLogger(TrainerCallback):
    def __init__(self, path):
        self.path, self._rows = str(path), 0

    def on_epoch_end(self, trainer, e):
        row = {"epoch": e.epoch, "loss": e.loss, "validation_loss": e.validation_loss, "lr": e.learning_rate,
               "seconds": e.seconds, **e.metrics}
        new = self._rows == 0
        with open(self.path, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(row))
            if new:
                w.writeheader()
            w.writerow(row)
        self._rows += 1


class CheckpointCallback(TrainerCallback):
    """Saves the model every ``every`` epochs (``best_only``: when validation loss improved)."""

    def __init__(self, folder, every: int = 1, best_only: bool = False):
        self.folder, self.every, self.best_only, self._best = Path(folder), every, best_only, math.inf

    def on_epoch_end(self, trainer, e):
        if (e.epoch + 1) % self.every:
            return
        score = e.validation_loss if e.validation_loss is not None else e.loss
        if self.best_only and score >= self._best:
            return
        self._best = min(self._best, score)
        self.folder.mkdir(parents=True, exist_ok=True)
        ikw.save_module(trainer.model, self.folder / ("best.ikw" if self.best_only else f"epoch-{e.epoch + 1}.ikw"))


class EarlyStopping(TrainerCallback):
    def __init__(self, patience: int, min_improvement: float = 0.0):
        self.patience, self.min_improvement, self._best, self._bad = patience, min_improvement, math.inf, 0

    def on_epoch_end(self, trainer, e):
        score = e.validation_loss if e.validation_loss is not None else e.loss
        if score < self._best - self.min_improvement:
            self._best, self._bad = score, 0
        else:
            self._bad += 1
            if self._bad >= self.patience:
                trainer.request_stop("early stopping")


class LearningRateCallback(TrainerCallback):
    def __init__(self, schedule: Schedule, per: str = "epoch"):
        self.schedule, self.per = schedule, per

    def on_epoch_end(self, trainer, e):
        if self.per == "epoch":
            self.schedule.apply(trainer.optimizer, e.epoch + 1)

    def on_batch_end(self, trainer, e):
        if self.per == "step":
            self.schedule.apply(trainer.optimizer, e.step + 1)


# --------------------------------------------------------------------------- out-of-memory policies
class OutOfMemoryPolicies:
    """``fail``: re-raise. ``split``: run the step again as several smaller parts with accumulated gradients."""
    default_name = "split"
    names = ("fail", "split")


# --------------------------------------------------------------------------- trainer
class Trainer:
    def __init__(self, model: torch.nn.Module, optimizer, loss: Optional[Callable] = None, *,
                 metrics: Sequence[Metric] = (), callbacks: Sequence[TrainerCallback] = (),
                 early_stopping_patience: Optional[int] = None, restore_best_weights: bool = True,
                 min_improvement: float = 0.0, scheduler: Optional[Schedule] = None, scheduler_per: str = "step",
                 max_gradient_norm: Optional[float] = None, sync=None, stop_folder: Optional[str] = None,
                 resume_from: Optional[str] = None, checkpoint_folder: Optional[str] = None,
                 checkpoint_every_epochs: int = 1, checkpoint_keep: int = 1,
                 out_of_memory_policy: str = OutOfMemoryPolicies.default_name, on_epoch: Optional[Callable] = None,
                 grad_accumulation: int = 1):
        self.model, self.optimizer, self.loss = model, optimizer, loss
        self.metrics, self.callbacks = list(metrics), list(callbacks)
        self.early_stopping_patience, self.restore_best_weights = early_stopping_patience, restore_best_weights
        self.min_improvement = min_improvement
        self.scheduler, self.scheduler_per = scheduler, scheduler_per
        self.max_gradient_norm = max_gradient_norm
        self.sync = sync
        self.stop_folder = Path(stop_folder) if stop_folder else None
        self.resume_from = Path(resume_from) if resume_from else None
        self.checkpoint_folder = Path(checkpoint_folder) if checkpoint_folder else None
        self.checkpoint_every_epochs, self.checkpoint_keep = checkpoint_every_epochs, checkpoint_keep
        if out_of_memory_policy not in OutOfMemoryPolicies.names:
            raise ValueError(f"unknown out-of-memory policy '{out_of_memory_policy}' (one of {OutOfMemoryPolicies.names})")
        self.out_of_memory_policy = out_of_memory_policy
        self.on_epoch = on_epoch
        self.grad_accumulation = max(1, grad_accumulation)
        self.global_step = 0
        self._stop_reason: Optional[str] = None
        if max_gradient_norm is not None and hasattr(optimizer, "max_grad_norm"):
            optimizer.max_grad_norm = max_gradient_norm
        self.device = next(model.parameters()).device

    # ------------------------------------------------------------------ control
    def request_stop(self, reason: str = "requested"):
        self._stop_reason = reason

    def _stop_requested(self) -> bool:
        if self._stop_reason:
            return True
        if self.stop_folder is not None and (self.stop_folder / "stop").exists():
            self._stop_reason = "stop file"
            return True
        return False

    # ------------------------------------------------------------------ one step
    def _forward_loss(self, x, y):
        if self.loss is None:
            return self.model.loss(x, y), None
        pred = self.model(x)
        return self.loss(pred, y), pred

    def _train_batch(self, x, y, parts: int = 1):
        """Forward + backward (+ update) of one batch, optionally split into ``parts`` along dim 0."""
        if parts == 1:
            loss, pred = self._forward_loss(x, y)
            if self.sync is not None:
                with self.sync.overlap():
                    loss.backward()
            else:
                loss.backward()
            return loss.detach(), pred
        total, n = 0.0, x.shape[0]
        bounds = [round(i * n / parts) for i in range(parts + 1)]
        for i in range(parts):
            xs, ys = x[bounds[i]:bounds[i + 1]], y[bounds[i]:bounds[i + 1]]
            if xs.shape[0] == 0:
                continue
            loss, _ = self._forward_loss(xs, ys)
            w = xs.shape[0] / n
            last = i == parts - 1
            if self.sync is not None and last:
                with self.sync.overlap():
                    (loss * w).backward()
            else:
                (loss * w).backward()
            total += float(loss.detach()) * w
        return torch.tensor(total, device=x.device), None

    def _step(self, x, y):
        try:
            loss, pred = self._train_batch(x, y)
        except torch.cuda.OutOfMemoryError:
            if self.out_of_memory_policy == "fail":
                raise
            self._zero_grad()
            torch.cuda.empty_cache()
            parts, loss, pred = 2, None, None
            while loss is None:
                try:
                    loss, pred = self._train_batch(x, y, parts)
                    Telemetry.publish(Level.TRAINING, "OutOfMemoryRecovered", parts=parts)
                except torch.cuda.OutOfMemoryError:
                    self._zero_grad()
                    torch.cuda.empty_cache()
                    parts *= 2
                    if parts > max(2, x.shape[0]):
                        raise
        if self.sync is not None:
            self.sync.reduce_and_step()
        else:
            if self.max_gradient_norm is not None and not hasattr(self.optimizer, "max_grad_norm"):
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_gradient_norm)
            self.optimizer.step()
        self._zero_grad()
        return loss, pred

    def _zero_grad(self):
        if self.sync is not None and hasattr(self.sync, "zero_grad"):
            self.sync.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=False)

    # ------------------------------------------------------------------ fit
    def fit(self, train: Iterable, epochs: int, validation: Optional[Iterable] = None) -> TrainingHistory:
        history = TrainingHistory()
        start_epoch, skip_steps = 0, 0
        best_state = None
        bad_epochs = 0
        if self.resume_from is not None:
            state = self.load_checkpoint(self.resume_from)
            if "epoch" in state:
                start_epoch, skip_steps = int(state["epoch"]), int(state.get("step_in_epoch", 0))
            else:
                # a checkpoint that only counts steps (the reference's layout): place it by the length of an epoch
                per_epoch = len(train) if hasattr(train, "__len__") else 0
                if per_epoch <= 0 and self.global_step > 0:
                    raise ValueError("this checkpoint records steps only; resuming it needs a training source with a length")
                start_epoch, skip_steps = (divmod(self.global_step, per_epoch) if per_epoch else (0, 0))
            if state.get("best_loss") is not None:
                history.best_loss = float(state["best_loss"])
            history.best_epoch = int(state.get("best_epoch", -1))
            bad_epochs = int(state.get("since_best", 0))
            best_state = state.get("_best_weights")
        self._early = (history, bad_epochs, best_state)
        for cb in self.callbacks:
            cb.on_train_begin(self)
        self.model.train()
        for epoch in range(start_epoch, epochs):
            t0 = time.perf_counter()
            loss_sum, n_batches, samples = 0.0, 0, 0
            metric_sums = {m.name: 0.0 for m in self.metrics}
            for step_in_epoch, (x, y) in enumerate(train):
                if skip_steps > 0:          # resumed: redraw the finished steps without training
                    skip_steps -= 1
                    continue
                x, y = x.to(self.device), y.to(self.device)
                if self.scheduler is not None and self.scheduler_per == "step":
                    self.scheduler.apply(self.optimizer, self.global_step)
                loss, pred = self._step(x, y)
                self.global_step += 1
                lv = float(loss)
                loss_sum += lv
                n_batches += 1
                samples += x.shape[0]
                if pred is not None:
                    with torch.no_grad():
                        for m in self.metrics:
                            metric_sums[m.name] += float(m.batch_mean(pred.detach(), y))
                ev = BatchCompleted(epoch=epoch, step=self.global_step - 1, loss=lv, size=int(x.shape[0]))
                Telemetry.publish_event(Level.BATCHES, ev)
                for cb in self.callbacks:
                    cb.on_batch_end(self, ev)
                if self._stop_requested():
                    if self.checkpoint_folder is not None or self.stop_folder is not None:
                        self.save_checkpoint(self.checkpoint_folder or self.stop_folder, epoch, step_in_epoch + 1)
                    history.stopped_by_request = self._stop_reason not in ("early stopping",)
                    break
            if self._stop_reason and self._stop_reason != "early stopping":
                break
            val = self.evaluate(validation) if validation is not None else None
            self.model.train()
            metrics = {k: v / max(1, n_batches) for k, v in metric_sums.items()}
            for m in self.metrics:
                if m.finalize:
                    metrics[m.name] = m.finalize(metrics[m.name])
            lr = getattr(self.optimizer, "lr", None) or self.optimizer.param_groups[0]["lr"]
            ev = EpochCompleted(epoch=epoch, loss=loss_sum / max(1, n_batches),
                                validation_loss=val.loss if val else None, metrics=metrics,
                                validation_metrics=val.metrics if val else {}, learning_rate=float(lr),
                                seconds=time.perf_counter() - t0, samples=samples)
            history.epochs.append(ev)
            Telemetry.publish_event(Level.TRAINING, ev)
            if self.on_epoch:
                self.on_epoch(ev)
            for cb in self.callbacks:
                cb.on_epoch_end(self, ev)
            if self.scheduler is not None and self.scheduler_per == "epoch":
                self.scheduler.apply(self.optimizer, epoch + 1)
            score = ev.validation_loss if ev.validation_loss is not None else ev.loss
            if score < history.best_loss - self.min_improvement:
                history.best_loss, history.best_epoch, bad_epochs = score, epoch, 0
                if self.early_stopping_patience is not None and self.restore_best_weights:
                    best_state = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
            else:
                bad_epochs += 1
            self._early = (history, bad_epochs, best_state)
            if self.checkpoint_folder is not None and (epoch + 1) % self.checkpoint_every_epochs == 0:
                self.save_checkpoint(self.checkpoint_folder, epoch + 1, 0)
            if self.early_stopping_patience is not None and bad_epochs >= self.early_stopping_patience:
                history.stopped_early = True
                break
            if self._stop_reason == "early stopping":
                history.stopped_early = True
                break
        if history.stopped_early and best_state is not None:
            self.model.load_state_dict(best_state)
        for cb in self.callbacks:
            cb.on_train_end(self, history)
        return history

    # ------------------------------------------------------------------ evaluate / predict
    @torch.no_grad()
    def evaluate(self, data: Iterable) -> EvaluationResult:
        was_training = self.model.training
        self.model.eval()
        loss_sum, n, samples = 0.0, 0, 0
        sums = {m.name: 0.0 for m in self.metrics}
        for x, y in data:
            x, y = x.to(self.device), y.to(self.device)
            loss, pred = self._forward_loss(x, y)
            loss_sum += float(loss)
            n += 1
            samples += x.shape[0]
            if pred is not None:
                for m in self.metrics:
                    sums[m.name] += float(m.batch_mean(pred, y))
        metrics = {k: v / max(1, n) for k, v in sums.items()}
        for m in self.metrics:
            if m.finalize:
                metrics[m.name] = m.finalize(metrics[m.name])
        if self.sync is not None and hasattr(self.sync, "sum_values"):
            tot = self.sync.sum_values([loss_sum, float(n)])
            loss_sum, n = tot[0], int(tot[1])
        self.model.train(was_training)
        return EvaluationResult(loss_sum / max(1, n), metrics, samples)

    @torch.no_grad()
    def predict(self, inputs: torch.Tensor, batch_size: int = 1024) -> torch.Tensor:
        was_training = self.model.training
        self.model.eval()
        outs = [self.model(inputs[i:i + batch_size].to(self.device)).cpu() for i in range(0, len(inputs), batch_size)]
        self.model.train(was_training)
        return torch.cat(outs)

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, folder, epoch: int, step_in_epoch: int) -> Path:
        folder = Path(folder)
        target = folder / f"checkpoint-{self.global_step}"
        tmp = folder / f".checkpoint-{self.global_step}.tmp"
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True)
        ikw.save_module(self.model, tmp / "model.ikw")
        if hasattr(self.optimizer, "state_dict"):
            state = self.optimizer.state_dict()
            if all(torch.is_tensor(v) for v in state.values()):
                save_file({k: v.float().contiguous() for k, v in state.items()}, tmp / "optimizer.safetensors",
                          metadata={"format": "idrak-optimizer", "optimizer": type(self.optimizer).__name__})
            else:
                torch.save(state, tmp / "optimizer.pt")
        history, since_best, best_state = getattr(self, "_early", (None, 0, None))
        state = {"format": TRAIN_STATE_FORMAT, "step": self.global_step,
                 "best_epoch": history.best_epoch if history is not None else -1, "since_best": int(since_best),
                 "dropout_draws": dropout_draws(self.model),
                 # beyond the reference's keys: where in the epoch the run stood, and how it was stopped
                 "epoch": epoch, "step_in_epoch": step_in_epoch,
                 "lr": float(getattr(self.optimizer, "lr", 0.0) or 0.0), "stop_reason": self._stop_reason}
        if history is not None and math.isfinite(history.best_loss):
            state["best_loss"] = history.best_loss
        if best_state is not None:
            # the weights of the best epoch so far, one flat fp32 entry per parameter / buffer, named by position
            save_file({str(i): v.detach().float().reshape(-1).contiguous().cpu() for i, v in enumerate(best_state.values())},
                      tmp / "best-weights.safetensors", metadata={"format": "idrak-best-weights"})
        torch.save({"cpu": torch.get_rng_state(),
                    "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else []}, tmp / "rng-state.pt")
        (tmp / "train-state.json").write_text(json.dumps(state, indent=2) + "\n")
        if target.exists():
            shutil.rmtree(target)
        os.replace(tmp, target)
        kept = sorted((p for p in folder.glob("checkpoint-*") if p.is_dir()),
                      key=lambda p: int(p.name.split("-")[1]))
        for old in kept[:-max(1, self.checkpoint_keep)]:
            shutil.rmtree(old, ignore_errors=True)
        return target

    def load_checkpoint(self, folder) -> dict:
        folder = Path(folder)
        if not (folder / "train-state.json").exists():
            cands = sorted((p for p in folder.glob("checkpoint-*") if p.is_dir()),
                           key=lambda p: int(p.name.split("-")[1]))
            if not cands:
                raise FileNotFoundError(f"no checkpoint in {folder}")
            folder = cands[-1]
        ikw.load_module(self.model, folder / "model.ikw")
        if (folder / "optimizer.safetensors").exists():
            with SafeTensorsReader.open(folder / "optimizer.safetensors") as r:
                self.optimizer.load_state_dict({k: r.read(k) for k in r.tensors})
        elif (folder / "optimizer.pt").exists():
            self.optimizer.load_state_dict(torch.load(folder / "optimizer.pt", weights_only=True))
        if hasattr(self.optimizer, "sync_master_from_params"):
            self.optimizer.sync_master_from_params()
        state = json.loads((folder / "train-state.json").read_text())
        fmt = state.get("format")
        if fmt is not None and not str(fmt).startswith("idrak-train-state/"):
            raise ValueError(f"{folder / 'train-state.json'}: format '{fmt}' is not a trainer state")
        if "step" not in state and "global_step" not in state:
            raise ValueError(f"{folder / 'train-state.json'} names no step")
        self.global_step = int(state["step"] if "step" in state else state["global_step"])
        draws = state.get("dropout_draws") or []
        if draws:
            restore_dropout_draws(self.model, draws, folder)
        if (folder / "rng-state.pt").exists():
            rng = torch.load(folder / "rng-state.pt", weights_only=True)
            torch.set_rng_state(rng["cpu"])
            if torch.cuda.is_available() and len(rng["cuda"]) == torch.cuda.device_count():
                torch.cuda.set_rng_state_all(rng["cuda"])
        if (folder / "best-weights.safetensors").exists():
            with SafeTensorsReader.open(folder / "best-weights.safetensors") as r:
                current = self.model.state_dict()
                if len(r.tensors) != len(current):
                    raise ValueError(f"{folder}: best weights hold {len(r.tensors)} tensors, the model {len(current)}")
                best = {}
                for i, (k, v) in enumerate(current.items()):
                    flat = r.read(str(i))
                    if flat.numel() != v.numel():
                        raise ValueError(f"{folder}: best weights entry {i} has {flat.numel()} values, '{k}' has {v.numel()}")
                    best[k] = flat.reshape(v.shape).to(v.dtype).to(v.device)
                state["_best_weights"] = best
        return state
