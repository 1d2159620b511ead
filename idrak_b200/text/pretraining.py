"""Pre-training over token files: staged curriculum, a draw order all ranks share, checkpoints that resume at
another world size.

    stages = [PretrainStage("web", ["web.tokens"], steps=1000, seq_len=1024),
              PretrainStage("code", ["code.tokens", "math.tokens"], steps=200, seq_len=1024, weights=[3, 1])]
    Pretrainer.train(model, PretrainOptions(stages=stages, global_batch=64, micro_batch=16, out_dir="run"))

The global batch of step ``t`` of stage ``s`` is a pure function of ``(seed, s, t)``: which file and which window
each of its sequences comes from. Rank ``r`` of ``W`` takes sequences ``[r B / W, (r + 1) B / W)``, so the same run
can continue on a different number of GPUs and still see the same data. Data parallelism uses the fused
reduce-scatter + AdamW + all-gather path (``parallel/dp.py``) on GPUs and a plain gradient all-reduce on CPU ranks.
A checkpoint folder ``checkpoint-STEP`` holds the model as a Hugging Face folder (fp32 safetensors),
``optimizer.safetensors`` (``step``, ``m.i``, ``v.i`` by parameter index) and ``train-state.json``.

Reference: Pretrainer.Train and its options (src/Idrak.Text/Pretraining.cs:346, :78), optimizer state file
(Pretraining.cs:1098-1140), token files (src/Idrak.Text/TokenFiles.cs).
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..formats.safetensors import load_file, save_file
from ..formats.tokens import TokenFile
from ..ops import FusedAdamW


@dataclass
class PretrainStage:
    name: str
    files: List[str]
    steps: int
    seq_len: int = 1024
    weights: Optional[List[float]] = None      # mixing weights of the files (default: by their number of windows)


@dataclass
class PretrainOptions:
    stages: List[PretrainStage] = field(default_factory=list)
    global_batch: int = 64                     # sequences per optimizer step over all ranks
    micro_batch: int = 16                      # sequences per forward / backward on one rank
    learning_rate: float = 6e-4
    min_lr_ratio: float = 0.1
    warmup_steps: int = 100
    weight_decay: float = 0.1
    betas: Tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    clip: float = 1.0
    seed: int = 0
    save_every: int = 0
    eval_every: int = 0
    eval_files: List[str] = field(default_factory=list)
    eval_batches: int = 8
    out_dir: Optional[str] = None
    resume_from: Optional[str] = None
    use_graph: bool = False
    dp_mode: str = "fused"                     # fused | nccl
    log_every: int = 10


@dataclass
class PretrainResult:
    steps: int = 0
    tokens: int = 0
    losses: List[float] = field(default_factory=list)
    eval_losses: List[Tuple[int, float]] = field(default_factory=list)
    checkpoints: List[str] = field(default_factory=list)
    tokens_per_second: float = 0.0


def draw_global_batch(files: Sequence[TokenFile], weights: Optional[Sequence[float]], seed: int, stage: int, step: int,
                      batch: int) -> List[Tuple[int, int]]:
    """``(file index, window index)`` of each sequence of the step's global batch."""
    rng = np.random.default_rng([int(seed), int(stage), int(step)])
    w = np.asarray(weights if weights is not None else [len(f) for f in files], dtype=np.float64)
    w = w / w.sum()
    which = rng.choice(len(files), size=batch, p=w)
    return [(int(f), int(rng.integers(0, len(files[int(f)])))) for f in which]


def lr_at(step: int, total: int, o: PretrainOptions) -> float:
    if step < o.warmup_steps:
        return o.learning_rate * (step + 1) / max(o.warmup_steps, 1)
    t = (step - o.warmup_steps) / max(total - o.warmup_steps, 1)
    floor = o.learning_rate * o.min_lr_ratio
    return floor + 0.5 * (o.learning_rate - floor) * (1.0 + math.cos(math.pi * min(t, 1.0)))


class Pretrainer:
    def __init__(self, model, options: PretrainOptions, group=None):
        self.model, self.o, self.group = model, options, group
        self.device = next(model.parameters()).device
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        o = options
        if o.global_batch % self.world or (o.global_batch // self.world) % o.micro_batch:
            raise ValueError(f"global_batch ({o.global_batch}) must divide into world ({self.world}) x micro_batch "
                             f"({o.micro_batch}) x accumulation")
        self.accumulation = o.global_batch // self.world // o.micro_batch
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.sync = None
        if self.world > 1 and self.device.type == "cuda":
            from ..parallel.dp import DataParallel
            self.sync = DataParallel(model, lr=o.learning_rate, betas=o.betas, eps=o.eps, weight_decay=o.weight_decay,
                                     max_grad_norm=o.clip, mode=o.dp_mode, group=group)
            self.optimizer = self.sync.optimizer
        else:
            if self.world > 1:
                for p in model.parameters():
                    dist.broadcast(p.data, src=0, group=group)
            self.optimizer = FusedAdamW(model.decay_groups(o.weight_decay), lr=o.learning_rate, betas=o.betas, eps=o.eps,
                                        weight_decay=o.weight_decay, max_grad_norm=o.clip)
        from ..training.step import TrainStep
        self.step_fn = TrainStep(model, self.optimizer, sync=self.sync, grad_accumulation=self.accumulation,
                                 use_graph=o.use_graph and self.device.type == "cuda", ignore_index=None,
                                 direct_grads=self.device.type == "cuda")
        self.step = 0
        self.result = PretrainResult()

    # ------------------------------------------------------------------ schedule
    def total_steps(self) -> int:
        return sum(s.steps for s in self.o.stages)

    def locate(self, step: int) -> Tuple[int, int]:
        """(stage index, step inside the stage) of a global step."""
        for i, s in enumerate(self.o.stages):
            if step < s.steps:
                return i, step
            step -= s.steps
        raise IndexError("step beyond the last stage")

    # ------------------------------------------------------------------ one step
    def _cpu_rank_step(self, micro: List[Tuple[torch.Tensor, torch.Tensor]]) -> float:
        """CPU ranks (gloo): accumulate, all-reduce the mean gradient, step."""
        self.optimizer.zero_grad()
        total = 0.0
        for x, y in micro:
            loss = self.model.loss(x, y) / len(micro)
            loss.backward()
            total += float(loss.detach())
        flat = torch.cat([p.grad.reshape(-1) for p in self.params])
        dist.all_reduce(flat, group=self.group)
        flat /= self.world
        off = 0
        for p in self.params:
            p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
            off += p.numel()
        self.optimizer.step()
        t = torch.tensor([total])
        dist.all_reduce(t, group=self.group)
        return float(t) / self.world

    def run_step(self, files: Sequence[TokenFile], stage_index: int, stage_step: int) -> float:
        o = self.o
        stage = o.stages[stage_index]
        draws = draw_global_batch(files, stage.weights, o.seed, stage_index, stage_step, o.global_batch)
        per_rank = o.global_batch // self.world
        mine = draws[self.rank * per_rank:(self.rank + 1) * per_rank]
        lr = lr_at(self.step, self.total_steps(), o)
        if hasattr(self.optimizer, "set_lr"):
            self.optimizer.set_lr(lr)
        else:
            self.optimizer.lr = lr
        micro = []
        for k in range(self.accumulation):
            part = mine[k * o.micro_batch:(k + 1) * o.micro_batch]
            xs, ys = zip(*(files[f].window(w) for f, w in part))
            micro.append((torch.stack(xs).int(), torch.stack(ys).int()))
        if self.world > 1 and self.device.type != "cuda":
            return self._cpu_rank_step(micro)
        losses = []
        for x, y in micro:
            loss = self.step_fn(x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True))
            losses.append(loss.detach().float().reshape(()).clone())
        mean = torch.stack(losses).mean()          # the step's loss: mean over micro-batches (and ranks)
        if self.world > 1:
            dist.all_reduce(mean, group=self.group)
            mean = mean / self.world
        return float(mean.item())

    @torch.no_grad()
    def evaluate(self, seq_len: int) -> float:
        o = self.o
        files = [TokenFile(p, seq_len) for p in o.eval_files]
        self.model.eval()
        total, n = 0.0, 0
        for b in range(o.eval_batches):
            draws = draw_global_batch(files, None, o.seed + 7919, 0, b, o.micro_batch)
            xs, ys = zip(*(files[f].window(w) for f, w in draws))
            x, y = torch.stack(xs).int().to(self.device), torch.stack(ys).int().to(self.device)
            total += float(self.model.loss(x, y))
            n += 1
        self.model.train()
        return total / max(n, 1)

    # ------------------------------------------------------------------ checkpoints
    def _canonical_optimizer_state(self) -> Dict[str, torch.Tensor]:
        """``step``, ``m.i``, ``v.i`` with ``i`` the index among the model's trainable parameters."""
        if self.sync is not None and self.sync.mode == "fused":
            return self.sync.optimizer_state()
        state = self.optimizer.state_dict()
        index = {id(p): i for i, p in enumerate(self.params)}
        out = {"step": state["step"]}
        for j, p in enumerate(self.optimizer.params):
            for key in ("m", "v"):
                if f"{key}.{j}" in state:
                    out[f"{key}.{index[id(p)]}"] = state[f"{key}.{j}"]
        return out

    def _load_canonical_optimizer_state(self, state: Dict[str, torch.Tensor]) -> None:
        if self.sync is not None and self.sync.mode == "fused":
            self.sync.load_optimizer_state(state)
            return
        index = {id(p): i for i, p in enumerate(self.params)}
        mine = {"step": state["step"]}
        for j, p in enumerate(self.optimizer.params):
            for key in ("m", "v"):
                k = f"{key}.{index[id(p)]}"
                if k in state:
                    mine[f"{key}.{j}"] = state[k]
        self.optimizer.load_state_dict(mine)

    def save_checkpoint(self, folder: str) -> None:
        state = self._canonical_optimizer_state()          # collective under fused data parallelism
        if self.rank == 0:
            from ..models.pretrained import save_huggingface
            Path(folder).mkdir(parents=True, exist_ok=True)
            save_huggingface(self.model, folder, dtype=torch.float32)
            save_file({k: v.float().cpu() for k, v in state.items()}, os.path.join(folder, "optimizer.safetensors"),
                      metadata={"format": "idrak-optimizer", "optimizer": "AdamW"})
            stage, stage_step = self.locate(self.step) if self.step < self.total_steps() else (len(self.o.stages), 0)
            with open(os.path.join(folder, "train-state.json"), "w") as f:
                json.dump({"step": self.step, "stage": stage, "stage_step": stage_step, "tokens": self.result.tokens,
                           "world": self.world, "seed": self.o.seed, "global_batch": self.o.global_batch}, f, indent=1)
            self.result.checkpoints.append(folder)
        if self.world > 1:
            dist.barrier(group=self.group)

    def load_checkpoint(self, folder: str) -> None:
        from ..models.checkpoint import from_hf_tensors, load_idrak_tensors
        tensors = load_file(os.path.join(folder, "model.safetensors"))
        style = "gpt2" if self.model.spec.learned_positions else "llama"
        load_idrak_tensors(self.model, from_hf_tensors(self.model.spec, tensors, style))   # copies in place
        if self.sync is not None and self.sync.mode == "fused":
            self.sync.refresh_master_from_parameters()
        self._load_canonical_optimizer_state(load_file(os.path.join(folder, "optimizer.safetensors")))
        with open(os.path.join(folder, "train-state.json")) as f:
            st = json.load(f)
        if st.get("global_batch", self.o.global_batch) != self.o.global_batch or st.get("seed", self.o.seed) != self.o.seed:
            raise ValueError("the checkpoint was written with another global batch or seed: the data order would differ")
        self.step, self.result.tokens = int(st["step"]), int(st.get("tokens", 0))

    # ------------------------------------------------------------------ the run
    def fit(self, progress: Optional[Callable[[int, float], None]] = None) -> PretrainResult:
        o, res = self.o, self.result
        if not o.stages:
            raise ValueError("no stages")
        if o.resume_from:
            self.load_checkpoint(o.resume_from)
        total = self.total_steps()
        self.model.train()
        opened: Dict[int, List[TokenFile]] = {}
        t0, tokens0 = time.perf_counter(), res.tokens
        while self.step < total:
            si, ss = self.locate(self.step)
            stage = o.stages[si]
            if si not in opened:
                opened = {si: [TokenFile(p, stage.seq_len) for p in stage.files]}
                for f in opened[si]:
                    if len(f) == 0:
                        raise ValueError(f"{f.path}: shorter than one window of {stage.seq_len + 1} tokens")
            loss = self.run_step(opened[si], si, ss)
            if not math.isfinite(loss):
                raise FloatingPointError(f"non-finite loss at step {self.step}")
            self.step += 1
            res.steps = self.step
            res.tokens += o.global_batch * stage.seq_len
            res.losses.append(loss)
            if progress and (self.step % max(o.log_every, 1) == 0 or self.step == total):
                progress(self.step, loss)
            if o.eval_files and o.eval_every and self.step % o.eval_every == 0:
                res.eval_losses.append((self.step, self.evaluate(stage.seq_len)))
            if o.out_dir and o.save_every and self.step % o.save_every == 0 and self.step < total:
                self.save_checkpoint(os.path.join(o.out_dir, f"checkpoint-{self.step}"))
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        res.tokens_per_second = (res.tokens - tokens0) / dt if dt > 0 else 0.0
        if o.out_dir:
            self.save_checkpoint(os.path.join(o.out_dir, f"checkpoint-{self.step}"))
        return res

    @staticmethod
    def train(model, options: PretrainOptions, group=None, progress=None) -> PretrainResult:
        return Pretrainer(model, options, group).fit(progress)
