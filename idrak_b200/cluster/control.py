"""Agreement between ranks at step boundaries: the step header, stop requests, pause / resume / stop by file.

* ``StepHeader``: every rank contributes (step, token count, loss x tokens, stop request, a hash of its parameter
  shapes); the reduced header tells every rank the global token count (for token-weighted gradients), whether
  anyone asked to stop, and whether the ranks run the same model - a mismatch is an error that says so.
* ``StopAgreement``: a stop asked for on any rank (signal, stop file, time budget) takes effect on all ranks at the
  same step boundary, because the flag travels with the header that is reduced anyway.
* ``ControlFileSteering``: rank 0 watches a small JSON file (``{"command": "pause" | "resume" | "stop"}``) and the
  command is broadcast, so an operator can steer a run without signals.

They work over ``torch.distributed`` (any backend) or over a simulator ``RankContext``.

Reference: AllReduceStopAgreement.cs, ControlFileSteering.cs, the gradient header (GradientReduction.cs:73-75,796-811).
"""
from __future__ import annotations

import json
import os
import time
import zlib
from dataclasses import dataclass
from typing import Iterable, Optional

import numpy as np


class ClusterRunStopped(Exception):
    """All ranks agreed to stop at this step boundary (checkpoint, then leave with exit code 0)."""


class HeaderMismatch(RuntimeError):
    pass


def _reduce(values: np.ndarray, op: str, ctx=None, group=None) -> np.ndarray:
    if ctx is not None:
        return ctx.all_reduce(values, op)
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return values
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=group)
    return t.cpu().numpy()


def shapes_hash(params: Iterable) -> int:
    """A 24-bit fingerprint of the parameter shapes (fits a float exactly)."""
    text = ";".join(",".join(str(d) for d in p.shape) for p in params)
    return zlib.crc32(text.encode()) & 0xFFFFFF


@dataclass
class ReducedHeader:
    step: int
    tokens: float
    mean_loss: float
    stop: bool
    ranks: int


class StepHeader:
    def __init__(self, model_hash: int = 0, ctx=None, group=None):
        self.model_hash, self.ctx, self.group = model_hash, ctx, group

    def exchange(self, step: int, tokens: float, loss: float, stop: bool = False) -> ReducedHeader:
        sums = _reduce(np.array([tokens, loss * tokens, 1.0]), "sum", self.ctx, self.group)
        # maxima carry what must be equal everywhere (value and its negation) and the stop flag
        maxima = _reduce(np.array([step, -step, self.model_hash, -self.model_hash, 1.0 if stop else 0.0]), "max",
                         self.ctx, self.group)
        if maxima[0] != -maxima[1]:
            raise HeaderMismatch(f"ranks disagree on the step: {int(-maxima[1])} to {int(maxima[0])} (this rank: {step})")
        if maxima[2] != -maxima[3]:
            raise HeaderMismatch("ranks hold models with different parameter shapes")
        total = float(sums[0])
        return ReducedHeader(step, total, float(sums[1]) / total if total > 0 else 0.0, bool(maxima[4] > 0), int(sums[2]))


class StopAgreement:
    def __init__(self, header: StepHeader, stop_file: Optional[str] = None, deadline: Optional[float] = None,
                 clock=time.monotonic):
        self.header, self.stop_file, self.deadline, self.clock = header, stop_file, deadline, clock
        self.requested = False
        self.reason: Optional[str] = None

    def request(self, reason: str = "requested") -> None:
        self.requested, self.reason = True, reason

    def _local(self) -> bool:
        if self.stop_file and os.path.exists(self.stop_file):
            self.request(f"stop file {self.stop_file}")
        if self.deadline is not None and self.clock() >= self.deadline:
            self.request("time budget")
        return self.requested

    def at_boundary(self, step: int, tokens: float = 1.0, loss: float = 0.0) -> ReducedHeader:
        """Call once per step on every rank; raises ``ClusterRunStopped`` on all of them together."""
        h = self.header.exchange(step, tokens, loss, self._local())
        if h.stop:
            raise ClusterRunStopped(f"stop agreed at step {step}" + (f" ({self.reason})" if self.reason else ""))
        return h


class ControlFileSteering:
    """Rank 0 reads the control file; everyone acts on the same command at the same boundary."""

    COMMANDS = {"run": 0, "resume": 0, "pause": 1, "stop": 2}

    def __init__(self, path: str, rank: int = 0, ctx=None, group=None, poll_seconds: float = 0.2, sleep=time.sleep):
        self.path, self.rank, self.ctx, self.group = path, rank, ctx, group
        self.poll_seconds, self.sleep = poll_seconds, sleep
        self.pauses = 0

    def _read(self) -> int:
        if self.rank != 0 or not os.path.exists(self.path):
            return 0
        try:
            with open(self.path, "r", encoding="utf-8") as f:
                cmd = json.load(f).get("command", "run")
        except (ValueError, OSError):
            return 0                      # a half-written file: look again at the next boundary
        if cmd not in self.COMMANDS:
            raise ValueError(f"{self.path}: unknown command '{cmd}' (run, pause, resume, stop)")
        return self.COMMANDS[cmd]

    def at_boundary(self, step: int) -> None:
        while True:
            code = int(_reduce(np.array([float(self._read())]), "max", self.ctx, self.group)[0])
            if code == 2:
                raise ClusterRunStopped(f"stop command in {self.path} at step {step}")
            if code == 0:
                return
            self.pauses += 1
            self.sleep(self.poll_seconds)
