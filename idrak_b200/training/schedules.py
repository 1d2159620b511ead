"""Learning-rate schedules: step, exponential, cosine, lambda, warm-up + cosine.

A schedule maps a step (or epoch) index to a learning rate; ``apply(optimizer, t)`` sets it on any
optimizer of this package or of ``torch.optim``.

Reference: LearningRateSchedules / Schedulers (src/Idrak.Abstraction/Training/LearningRateSchedules.cs,
Schedulers.cs); the GPT sample's cosine with linear warm-up
(samples/Idrak.Samples.GptTraining/Program.cs:183-218).
"""
from __future__ import annotations

import math
from typing import Callable


class Schedule:
    def __init__(self, base_lr: float):
        self.base_lr = base_lr

    def lr(self, t: int) -> float:
        return self.base_lr

    def apply(self, optimizer, t: int) -> float:
        lr = self.lr(t)
        if hasattr(optimizer, "set_lr"):
            optimizer.set_lr(lr)
        else:
            for g in optimizer.param_groups:
                g["lr"] = lr
        return lr


class StepDecay(Schedule):
    def __init__(self, base_lr: float, step_size: int, gamma: float = 0.1):
        super().__init__(base_lr)
        self.step_size, self.gamma = step_size, gamma

    def lr(self, t):
        return self.base_lr * self.gamma ** (t // self.step_size)


class ExponentialDecay(Schedule):
    def __init__(self, base_lr: float, gamma: float):
        super().__init__(base_lr)
        self.gamma = gamma

    def lr(self, t):
        return self.base_lr * self.gamma ** t


class Cosine(Schedule):
    def __init__(self, base_lr: float, total: int, min_lr: float = 0.0):
        super().__init__(base_lr)
        self.total, self.min_lr = max(1, total), min_lr

    def lr(self, t):
        p = min(1.0, t / self.total)
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * p))


class WarmupCosine(Schedule):
    """Linear warm-up over ``warmup`` steps, then cosine decay to ``min_lr`` at ``total``."""

    def __init__(self, base_lr: float, warmup: int, total: int, min_lr: float = 0.0):
        super().__init__(base_lr)
        self.warmup, self.total, self.min_lr = warmup, max(total, warmup + 1), min_lr

    def lr(self, t):
        if t < self.warmup:
            return self.base_lr * (t + 1) / self.warmup
        p = min(1.0, (t - self.warmup) / (self.total - self.warmup))
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * p))


class Lambda(Schedule):
    def __init__(self, base_lr: float, fn: Callable[[int], float]):
        super().__init__(base_lr)
        self.fn = fn

    def lr(self, t):
        return self.base_lr * self.fn(t)


SCHEDULES = {"constant": Schedule, "step": StepDecay, "exponential": ExponentialDecay, "cosine": Cosine,
             "warmup-cosine": WarmupCosine, "lambda": Lambda}
