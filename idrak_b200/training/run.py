"""A training run as one object: everything ``Trainer`` takes plus what ``fit`` takes, with the trainer's defaults.
``dataclasses.replace(run, max_gradient_norm=0.5)`` makes a variant that differs in one setting.

    run = TrainingRun(model=model, loss=losses.sparse_cross_entropy, optimizer=lambda p: torch.optim.AdamW(p, 3e-3),
                      train=loader, epochs=40, validation=held_out, metrics=[Metric.accuracy()], max_gradient_norm=1.0)
    history = run.fit()

Reference: TrainingRun (src/Idrak/Training/TrainingRun.cs:36: the parameter-object form of Trainer plus Fit).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence

import torch

from .trainer import Metric, OutOfMemoryPolicies, Trainer, TrainerCallback, TrainingHistory


@dataclass
class TrainingRun:
    model: torch.nn.Module
    loss: Callable
    optimizer: Callable[[Iterable[torch.nn.Parameter]], object]      # built from the model's trainable parameters
    train: Iterable
    epochs: int
    validation: Optional[Iterable] = None
    scheduler: Optional[Callable[[object], object]] = None            # built from the optimizer
    scheduler_per: str = "step"
    metrics: Sequence[Metric] = ()
    callbacks: Sequence[TrainerCallback] = ()
    early_stopping_patience: Optional[int] = None
    restore_best_weights: bool = True
    min_improvement: float = 0.0
    max_gradient_norm: Optional[float] = None
    sync: object = None
    stop_folder: Optional[str] = None
    resume_from: Optional[str] = None
    checkpoint_folder: Optional[str] = None
    checkpoint_every_epochs: int = 1
    checkpoint_keep: int = 1
    out_of_memory_policy: str = OutOfMemoryPolicies.default_name
    grad_accumulation: int = 1
    trainer: Optional[Trainer] = field(default=None, init=False, repr=False, compare=False)

    def build(self) -> Trainer:
        opt = self.optimizer([p for p in self.model.parameters() if p.requires_grad])
        sched = self.scheduler(opt) if self.scheduler is not None else None
        self.trainer = Trainer(self.model, opt, self.loss, metrics=self.metrics, callbacks=self.callbacks,
                               early_stopping_patience=self.early_stopping_patience,
                               restore_best_weights=self.restore_best_weights, min_improvement=self.min_improvement,
                               scheduler=sched, scheduler_per=self.scheduler_per, max_gradient_norm=self.max_gradient_norm,
                               sync=self.sync, stop_folder=self.stop_folder, resume_from=self.resume_from,
                               checkpoint_folder=self.checkpoint_folder, checkpoint_every_epochs=self.checkpoint_every_epochs,
                               checkpoint_keep=self.checkpoint_keep, out_of_memory_policy=self.out_of_memory_policy,
                               grad_accumulation=self.grad_accumulation)
        return self.trainer

    def fit(self) -> TrainingHistory:
        return self.build().fit(self.train, self.epochs, self.validation)
