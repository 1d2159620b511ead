"""Supervised fine-tuning with LoRA / DoRA adapters over a frozen base (bf16, int8 or int4).

    result = FineTuner.train(model, tokenizer, examples, options=FineTuningOptions(base="int4"), out_dir="out")

Examples are dicts: ``{"text"}`` (every token is trained), ``{"prompt", "response"}`` (only the response is trained)
or ``{"messages": [...]}`` (only assistant turns are trained; rendered through the chat template). Sequences are
packed first-fit into rows of at most ``max_length`` tokens; a batch holds rows up to ``batch_tokens``. Inside a
packed row attention stays within each sequence and positions restart. The step runs the frozen projections on
the dequant-fused tcgen05 GEMM with the low-rank term added, adapters only are optimised (fused AdamW), gradients
are clipped at 1.0, a non-finite loss skips the step, and the result is written as a PEFT adapter folder.

Reference: FineTuner.Train and FineTuningOptions (src/Idrak.Text/FineTuning.cs:1176, :767-1007), ChatTranscriptEncoder
(src/Idrak.Text/ChatTranscriptEncoder.cs:169), preference losses (src/Idrak.Text/FineTuningLosses.cs).
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import random
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..adapters.lora import DEFAULT_TARGETS, add_adapters, adapter_parameters
from ..adapters.peft import load_adapters, save_adapters
from ..ops import FusedAdamW
from .chat import ChatTemplate

IGNORE = -100


@dataclass
class FineTuningOptions:
    rank: int = 16
    alpha: float = 32.0
    targets: Tuple[str, ...] = tuple(DEFAULT_TARGETS)
    dora: bool = False
    rslora: bool = False
    base: str = "bf16"                   # how the frozen base is held: bf16 | int8 | int4 | fp8 (e4m3 codes, the forward
                                         # products on the 8-bit tensor-core path, input gradients in bf16)
    learning_rate: float = 2e-4
    weight_decay: float = 0.0
    warmup_fraction: float = 0.03
    schedule: str = "cosine"             # cosine | linear | constant
    clip: float = 1.0
    epochs: int = 1
    max_steps: int = 0                   # 0 = run the epochs out
    batch_tokens: int = 4096
    max_length: int = 2048
    packing: bool = True
    accumulation: int = 1
    loss_chunk_rows: int = 512
    non_finite_steps: int = 8            # give up after this many skipped steps in a row
    data_parallel: str = "fused"         # with several ranks on GPUs: fused (peer-memory reduce-scatter + sharded AdamW +
                                         # all-gather kernels) | nccl (the same buckets over NCCL) | flat (one all-reduce)
    capture_graph: bool = False          # one GPU, sft loss, no accumulation: pad every batch to one length, record
                                         # forward + backward + update once as a CUDA graph and replay it per step
    checkpoint_blocks: bool = False      # recompute block activations in backward
    activation_ladder: bool = True       # estimate activation memory before the first step, step down on out-of-memory
    loss: str = "sft"                    # sft | dpo | orpo | simpo (or a name registered in PREFERENCE_LOSSES)
    dpo_beta: float = 0.1
    orpo_lambda: float = 0.1             # weight of ORPO's odds-ratio term
    simpo_beta: float = 2.0              # SimPO's reward scale and target margin
    simpo_gamma: float = 1.0
    save_every: int = 0                  # steps; 0 = only at the end
    eval_every: int = 0
    seed: int = 0
    resume_from: Optional[str] = None


@dataclass
class FineTuningResult:
    steps: int = 0
    tokens: int = 0
    losses: List[float] = field(default_factory=list)
    eval_losses: List[Tuple[int, float]] = field(default_factory=list)
    skipped_steps: int = 0
    graph_replays: int = 0               # steps that were a replay of the recorded graph (``capture_graph``)
    adapter_folder: Optional[str] = None
    activation_policy: str = "held"


# ------------------------------------------------------------------ examples -> token rows
def encode_example(example: Dict[str, Any], tokenizer, template: Optional[ChatTemplate] = None,
                   max_length: int = 2048) -> Tuple[List[int], List[bool]]:
    """Token ids of one example and, per token, whether it is a training target."""
    eos = list(tokenizer.eos_token_ids[:1])
    if "messages" in example:
        template = template or ChatTemplate.for_tokenizer(tokenizer)
        ids: List[int] = []
        train: List[bool] = []
        msgs = example["messages"]
        done = 0
        for i, m in enumerate(msgs):
            if m.get("role") != "assistant":
                continue
            # text up to this assistant turn (with the generation prompt) is context; the turn itself is trained
            before = tokenizer.encode(template.render(msgs[:i], add_generation_prompt=True), add_special_tokens=False)
            upto = tokenizer.encode(template.render(msgs[: i + 1], add_generation_prompt=False), add_special_tokens=False)
            if upto[: len(before)] != before:          # the template rewrites history: fall back to a prefix match
                k = 0
                while k < min(len(before), len(upto)) and before[k] == upto[k]:
                    k += 1
                before = upto[:k]
            ids += upto[done:]
            train += [False] * (len(before) - done) + [True] * (len(upto) - len(before))
            done = len(upto)
        if not ids:
            raise ValueError("a 'messages' example needs at least one assistant turn")
    elif "prompt" in example:
        p = tokenizer.encode(example["prompt"], add_special_tokens=True)
        r = tokenizer.encode(example.get("response", example.get("completion", "")), add_special_tokens=False) + eos
        ids, train = p + r, [False] * len(p) + [True] * len(r)
    elif "text" in example:
        ids = tokenizer.encode(example["text"], add_special_tokens=True) + eos
        train = [True] * len(ids)
    else:
        raise ValueError("an example needs 'text', 'prompt' + 'response', or 'messages'")
    return ids[:max_length], train[:max_length]


@dataclass
class PackedBatch:
    ids: torch.Tensor            # int32 [1, T]
    targets: torch.Tensor        # int64 [1, T]; IGNORE where not trained
    positions: torch.Tensor      # int32 [T]
    spans: List[Tuple[int, int]]
    trained_tokens: int


def pack_batches(encoded: Sequence[Tuple[List[int], List[bool]]], batch_tokens: int, max_length: int,
                 packing: bool = True) -> List[PackedBatch]:
    """First-fit rows of at most ``max_length`` tokens, grouped into batches of at most ``batch_tokens``; every batch
    is one packed row of sequences (``spans``), which is how the decoder takes them."""
    rows: List[List[int]] = []          # indices of examples per row
    room: List[int] = []
    for i, (ids, _) in enumerate(encoded):
        n = len(ids)
        if n < 2:
            continue
        placed = False
        if packing:
            for r in range(len(rows)):
                if room[r] >= n:
                    rows[r].append(i)
                    room[r] -= n
                    placed = True
                    break
        if not placed:
            rows.append([i])
            room.append(max_length - n)
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_tokens = 0
    for r, members in enumerate(rows):
        used = max_length - room[r]
        if cur and cur_tokens + used > batch_tokens:
            batches.append(cur)
            cur, cur_tokens = [], 0
        cur += members
        cur_tokens += used
    if cur:
        batches.append(cur)
    out = []
    for members in batches:
        ids_all, tgt_all, pos_all, spans = [], [], [], []
        trained = 0
        for i in members:
            ids, train = encoded[i]
            lo = len(ids_all)
            ids_all += ids
            # next-token targets inside the sequence; its last token predicts nothing
            tgt = [ids[j + 1] if train[j + 1] else IGNORE for j in range(len(ids) - 1)] + [IGNORE]
            trained += sum(1 for t in tgt if t != IGNORE)
            tgt_all += tgt
            pos_all += list(range(len(ids)))
            spans.append((lo, lo + len(ids)))
        # kernels want the packed length to be a multiple of 8: pad with an untrained tail sequence
        pad = (-len(ids_all)) % 8
        if pad:
            lo = len(ids_all)
            ids_all += [0] * pad
            tgt_all += [IGNORE] * pad
            pos_all += list(range(pad))
            spans.append((lo, lo + pad))
        out.append(PackedBatch(torch.tensor([ids_all], dtype=torch.int32), torch.tensor([tgt_all], dtype=torch.int64),
                               torch.tensor(pos_all, dtype=torch.int32), spans, trained))
    return out


def _lr_at(step: int, total: int, o: FineTuningOptions) -> float:
    warm = max(int(total * o.warmup_fraction), 1)
    if step < warm:
        return o.learning_rate * (step + 1) / warm
    if o.schedule == "constant" or total <= warm:
        return o.learning_rate
    t = (step - warm) / max(total - warm, 1)
    if o.schedule == "linear":
        return o.learning_rate * max(0.0, 1.0 - t)
    return o.learning_rate * 0.5 * (1.0 + math.cos(math.pi * min(t, 1.0)))


@contextlib.contextmanager
def adapters_disabled(model):
    """Run the frozen base alone (the reference policy of preference losses)."""
    held = []
    for mod in model.modules():
        if getattr(mod, "adapters", None) is not None:
            held.append((mod, mod.adapters))
            mod.adapters = None
    try:
        yield
    finally:
        for mod, a in held:
            mod.adapters = a


def sequence_logprobs(model, batch: PackedBatch, device, mean: bool = False) -> torch.Tensor:
    """Sum (or, with ``mean``, the per-token mean) of the trained tokens' log-probabilities of every sequence of a
    packed batch ``[len(spans)]``."""
    logits = model(batch.ids.to(device), batch.positions.to(device), spans=batch.spans)[0].float()
    lp = torch.log_softmax(logits, -1)
    tgt = batch.targets[0].to(device)
    keep = tgt != IGNORE
    tok = lp.gather(1, tgt.clamp(min=0)[:, None])[:, 0] * keep
    if mean:
        return torch.stack([tok[lo:hi].sum() / keep[lo:hi].sum().clamp(min=1) for lo, hi in batch.spans])
    return torch.stack([tok[lo:hi].sum() for lo, hi in batch.spans])


# --------------------------------------------------------------------------- preference losses
# Each takes (tuner, batch) with the chosen answer as sequence 0 and the rejected one as sequence 1 of the batch and
# returns a scalar. Registered by name so an application can add its own (the reference's PreferenceLosses registry,
# src/Idrak.Text/FineTuningLosses.cs:560-660).
def _dpo_loss(tuner, b):
    policy = sequence_logprobs(tuner.model, b, tuner.device)
    with torch.no_grad(), adapters_disabled(tuner.model):
        ref = sequence_logprobs(tuner.model, b, tuner.device)
    margin = (policy[0] - policy[1]) - (ref[0] - ref[1])
    return -torch.nn.functional.logsigmoid(tuner.o.dpo_beta * margin)


def orpo_from_means(chosen_mean: torch.Tensor, rejected_mean: torch.Tensor, lam: float) -> torch.Tensor:
    """Odds-ratio preference optimisation (Hong et al. 2024) from the answers' mean token log-probabilities a < 0:
    ``-a_c - lam * log sigmoid(log odds_c - log odds_r)`` with ``log odds = a - log(1 - exp a)``; no reference model."""
    def log_odds(a):
        return a - torch.log(1.0 - torch.exp(a) + 1e-7)
    return -chosen_mean - lam * torch.nn.functional.logsigmoid(log_odds(chosen_mean) - log_odds(rejected_mean))


def simpo_from_means(chosen_mean: torch.Tensor, rejected_mean: torch.Tensor, beta: float, gamma: float) -> torch.Tensor:
    """Simple preference optimisation (Meng et al. 2024): ``-log sigmoid(beta (a_c - a_r) - gamma)`` with a the mean
    token log-probability of an answer (a length-normalised reward) and gamma a target margin; no reference model."""
    return -torch.nn.functional.logsigmoid(beta * (chosen_mean - rejected_mean) - gamma)


def _orpo_loss(tuner, b):
    if tuner.o.orpo_lambda < 0:
        raise ValueError("orpo_lambda must not be negative")
    means = sequence_logprobs(tuner.model, b, tuner.device, mean=True)
    return orpo_from_means(means[0], means[1], tuner.o.orpo_lambda)


def _simpo_loss(tuner, b):
    if tuner.o.simpo_beta <= 0:
        raise ValueError("simpo_beta must be positive")
    means = sequence_logprobs(tuner.model, b, tuner.device, mean=True)
    return simpo_from_means(means[0], means[1], tuner.o.simpo_beta, tuner.o.simpo_gamma)


PREFERENCE_LOSSES: Dict[str, Callable] = {"dpo": _dpo_loss, "orpo": _orpo_loss, "simpo": _simpo_loss}


class FineTuner:
    """Drives the adapter training loop; ``FineTuner.train`` is the one-call form."""

    def __init__(self, model, tokenizer, options: Optional[FineTuningOptions] = None, group=None):
        self.model, self.tokenizer = model, tokenizer
        self.o = options or FineTuningOptions()
        self.group = group
        self.device = next(model.parameters()).device
        o = self.o
        if o.base in ("int8", "int4", "fp8") and self.device.type == "cuda":
            from ..quant import quantize_model
            quantize_model(model, o.base)
        elif o.base not in ("bf16", "float32", "int8", "int4", "fp8"):
            raise ValueError(f"unknown base format '{o.base}' (bf16, int8, int4, fp8)")
        if o.resume_from:          # the checkpoint's adapters come first: the optimizer is built over them
            load_adapters(model, o.resume_from)
        has = any(getattr(m, "adapters", None) is not None for m in model.modules())
        if has:
            self.params = adapter_parameters(model)
        else:
            # the adapters' initial values are a function of the seed, not of what else drew random numbers before
            devices = [self.device] if self.device.type == "cuda" else []
            with torch.random.fork_rng(devices=devices):
                torch.manual_seed(o.seed)
                self.params = add_adapters(model, o.rank, o.alpha, o.targets, dora=o.dora, rslora=o.rslora)
        for p in self.params:
            p.requires_grad_(True)
        model.checkpoint_blocks = o.checkpoint_blocks
        model.loss_chunk_rows = o.loss_chunk_rows
        self.sync = None
        many = dist.is_initialized() and dist.get_world_size(group) > 1
        if many and self.device.type == "cuda" and o.data_parallel in ("fused", "nccl"):
            # adapter gradients go through the bucketed reduce-scatter, the sharded AdamW and the all-gather of the
            # data-parallel engine, overlapped with the backward pass; the header carries token counts and the
            # non-finite-loss agreement
            from ..parallel.dp import DataParallel
            self.sync = DataParallel(model, lr=o.learning_rate, weight_decay=o.weight_decay, max_grad_norm=o.clip,
                                     mode=o.data_parallel, group=group, bucket_mb=8.0)
            self.optimizer = self.sync.optimizer
        else:
            if many:        # one all-reduce per step keeps equal weights equal: start them equal
                with torch.no_grad():
                    for p in self.params:
                        dist.broadcast(p.data, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                       group=group)
            self.optimizer = FusedAdamW([{"params": self.params, "weight_decay": o.weight_decay}], lr=o.learning_rate,
                                        weight_decay=o.weight_decay, max_grad_norm=o.clip)
        self.template = ChatTemplate.for_tokenizer(tokenizer)
        self.step = 0
        self.result = FineTuningResult()
        self.activation_policy = "checkpoint_blocks" if o.checkpoint_blocks else "held"

    # ------------------------------------------------------------------ activation memory
    def plan_activation_memory(self, tokens: int) -> str:
        """Pick the first rung of the ladder that fits the free memory for steps of ``tokens`` tokens."""
        from . import activation_memory as am
        if not self.o.activation_ladder:
            return self.activation_policy
        est = am.choose_policy(self.model.spec, tokens, am.free_device_bytes(self.device), adapter_rank=self.o.rank,
                               start=self.activation_policy)
        self.activation_policy = est.policy
        am.apply_policy(self.model, est.policy)
        self.result.activation_policy = est.policy
        return est.policy

    def _step_down(self) -> bool:
        """After an out-of-memory step: move to the next rung (False when there is none)."""
        from . import activation_memory as am
        nxt = am.next_rung(self.activation_policy) if self.o.activation_ladder else None
        if nxt is None:
            return False
        self.activation_policy = nxt
        am.apply_policy(self.model, nxt)
        self.result.activation_policy = nxt
        self.optimizer.zero_grad()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        return True

    # ------------------------------------------------------------------ data
    def batches(self, examples: Iterable[Dict[str, Any]]) -> List[PackedBatch]:
        o = self.o
        if o.loss in PREFERENCE_LOSSES:
            return self._preference_batches(examples)
        if o.loss != "sft":
            raise ValueError(f"unknown loss '{o.loss}'; known: sft, {', '.join(sorted(PREFERENCE_LOSSES))}")
        enc = [encode_example(e, self.tokenizer, self.template, o.max_length) for e in examples]
        return pack_batches(enc, o.batch_tokens, o.max_length, o.packing)

    def _preference_batches(self, examples) -> List[PackedBatch]:
        o, out = self.o, []
        for e in examples:            # one batch per pair: [chosen, rejected] packed in one row
            pair = [encode_example({"prompt": e["prompt"], "response": e[k]}, self.tokenizer, self.template, o.max_length)
                    for k in ("chosen", "rejected")]
            out += pack_batches(pair, 2 * o.max_length, o.max_length, packing=False)
        return out

    # ------------------------------------------------------------------ losses
    # ------------------------------------------------------------------ graph-recorded step
    def _graph_eligible(self) -> bool:
        o = self.o
        return (o.capture_graph and self.device.type == "cuda" and self.sync is None and o.accumulation == 1
                and o.loss == "sft" and not o.checkpoint_blocks)

    def _graph_setup(self, batches: Sequence[PackedBatch]) -> None:
        """Static device buffers of one padded length and a ``TrainStep`` that records the step over them. A batch
        shorter than that length gets an untrained tail that is a sequence of its own (it attends to nothing else and
        nothing attends to it)."""
        from ..training.step import TrainStep
        T = (max(b.ids.numel() for b in batches) + 7) // 8 * 8
        dev = self.device
        self._g_len = T
        self._g_positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self._g_row_start = torch.zeros((1, T), dtype=torch.int32, device=dev)
        pin = dict(pin_memory=True)
        self._g_host = (torch.zeros((1, T), dtype=torch.int32, **pin), torch.zeros((1, T), dtype=torch.int32, **pin),
                        torch.zeros(T, dtype=torch.int32, **pin), torch.zeros((1, T), dtype=torch.int32, **pin))

        def loss_fn(model, ids, targets):
            return model.loss(ids, targets, self._g_positions, ignore_index=IGNORE, spans=self._g_row_start)

        self._g_step = TrainStep(self.model, self.optimizer, use_graph=True, loss_fn=loss_fn, direct_grads=False)

    def _graph_step(self, b: PackedBatch) -> float:
        """One recorded step on batch ``b``: four small host-to-device copies, one replay, one loss read."""
        from ..ops.attention import row_starts_from_spans
        T, n = self._g_len, b.ids.numel()
        ids_h, tg_h, pos_h, rs_h = self._g_host
        ids_h.zero_()
        tg_h.fill_(IGNORE)
        pos_h.zero_()
        ids_h[0, :n] = b.ids.reshape(-1)
        tg_h[0, :n] = b.targets.reshape(-1).to(torch.int32)
        pos_h[:n] = b.positions.reshape(-1)
        spans = list(b.spans)
        if n < T:
            pos_h[n:] = torch.arange(T - n, dtype=torch.int32)
            spans.append((n, T))
        rs_h.copy_(row_starts_from_spans(spans, 1, T))
        self._g_positions.copy_(pos_h, non_blocking=True)
        self._g_row_start.copy_(rs_h, non_blocking=True)
        return self._g_step.step_from_host(ids_h, tg_h)

    def batch_loss(self, b: PackedBatch) -> torch.Tensor:
        dev = self.device
        if self.o.loss in PREFERENCE_LOSSES:
            if len(b.spans) < 2:          # chosen, rejected (and possibly an untrained padding tail)
                raise ValueError(f"the '{self.o.loss}' loss needs pairs: examples with 'prompt', 'chosen' and 'rejected'")
            return PREFERENCE_LOSSES[self.o.loss](self, b)
        return self.model.loss(b.ids.to(dev), b.targets.to(dev), b.positions.to(dev), ignore_index=IGNORE, spans=b.spans)

    @torch.no_grad()
    def evaluate(self, batches: Sequence[PackedBatch]) -> float:
        self.model.eval()
        total, count = 0.0, 0
        for b in batches:
            n = max(b.trained_tokens, 1)
            total += float(self.batch_loss(b)) * n
            count += n
        self.model.train()
        return total / max(count, 1)

    # ------------------------------------------------------------------ the loop
    def _reduce_grads(self) -> None:
        if self.group is None and not (dist.is_initialized() and dist.get_world_size() > 1):
            return
        world = dist.get_world_size(self.group)
        flat = torch.cat([p.grad.reshape(-1).float() for p in self.params if p.grad is not None])
        dist.all_reduce(flat, group=self.group)
        flat /= world
        off = 0
        for p in self.params:
            if p.grad is not None:
                p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
                off += p.numel()

    def fit(self, train: Sequence[Dict[str, Any]], evaluation: Optional[Sequence[Dict[str, Any]]] = None,
            out_dir: Optional[str] = None, progress: Optional[Callable[[int, float], None]] = None) -> FineTuningResult:
        o, res = self.o, self.result
        batches = self.batches(train)
        if not batches:
            raise ValueError("no trainable examples")
        eval_batches = self.batches(evaluation) if evaluation else []
        per_epoch = math.ceil(len(batches) / o.accumulation)
        total = o.max_steps if o.max_steps > 0 else per_epoch * o.epochs
        if o.resume_from:
            self.load_checkpoint(o.resume_from)
        rng = random.Random(o.seed)
        order: List[int] = []
        self.model.train()
        self.plan_activation_memory(max(b.ids.numel() for b in batches))
        bad_streak = 0
        cursor = self.step * o.accumulation
        graphed = self._graph_eligible()
        if graphed:
            self._graph_setup(batches)
        res.graph_replays = 0
        while self.step < total:
            while len(order) <= cursor + o.accumulation:       # the draw order is a pure function of the seed
                epoch_order = list(range(len(batches)))
                rng.shuffle(epoch_order)
                order += epoch_order
            group = [batches[order[cursor + k]] for k in range(o.accumulation)]
            cursor += o.accumulation
            tokens = sum(max(b.trained_tokens, 1) for b in group)
            if graphed:
                # the recorded step holds forward, backward, clip and update; a non-finite gradient norm makes the
                # update kernel leave the weights alone, so a bad step is skipped on the device and counted here
                self.optimizer.set_lr(_lr_at(self.step, total, o))
                value = self._graph_step(group[0])
                res.graph_replays = self._g_step.replays
                if not math.isfinite(value):
                    res.skipped_steps += 1
                    bad_streak += 1
                    if bad_streak >= o.non_finite_steps:
                        raise FloatingPointError(f"{bad_streak} steps in a row had a non-finite loss")
                    continue
                bad_streak = 0
                self.step += 1
                res.steps, res.tokens = self.step, res.tokens + tokens
                res.losses.append(value)
                if progress:
                    progress(self.step, value)
                if eval_batches and o.eval_every and self.step % o.eval_every == 0:
                    res.eval_losses.append((self.step, self.evaluate(eval_batches)))
                    self.model.train()
                if out_dir and o.save_every and self.step % o.save_every == 0:
                    self.save_checkpoint(os.path.join(out_dir, f"checkpoint-{self.step}"))
                continue
            if self.sync is not None:
                self.sync.zero_grad()
            else:
                self.optimizer.zero_grad()
            loss_value, finite = 0.0, True
            try:
                for i, b in enumerate(group):
                    w = max(b.trained_tokens, 1) / tokens          # token-weighted mean over the accumulated batches
                    loss = self.batch_loss(b)
                    value = float(loss.detach())                   # the one host read per batch
                    if not math.isfinite(value):
                        finite = False
                    if self.sync is None:
                        if not finite:
                            break
                        (loss * w).backward()
                        loss_value += value * w
                        continue
                    # several ranks: nobody may leave the step alone. Every rank reaches the header before the last
                    # backward; a non-finite loss anywhere makes the header's loss non-finite everywhere.
                    if finite:
                        loss_value += value * w
                    if i + 1 < len(group):
                        if finite:
                            (loss * w).backward()
                        continue
                    header = self.sync.step_header(tokens, loss_value if finite else float("nan"))
                    agreed = float(header["loss"])                 # the ranks' token-weighted mean loss
                    if not math.isfinite(agreed):
                        finite = False
                        break
                    with self.sync.overlap():
                        (loss * w).backward()
                    loss_value = agreed
            except torch.OutOfMemoryError:
                loss = None
                if not self._step_down():
                    raise
                cursor -= o.accumulation                           # the same batches again on the next rung
                continue
            if not finite:
                res.skipped_steps += 1
                bad_streak += 1
                if bad_streak >= o.non_finite_steps:
                    raise FloatingPointError(f"{bad_streak} steps in a row had a non-finite loss")
                continue
            bad_streak = 0
            self.optimizer.lr = _lr_at(self.step, total, o)
            if self.sync is not None:
                self.sync.reduce_and_step()
            else:
                self._reduce_grads()
                self.optimizer.step()
            self.step += 1
            res.steps, res.tokens = self.step, res.tokens + tokens
            res.losses.append(loss_value)
            if progress:
                progress(self.step, loss_value)
            if eval_batches and o.eval_every and self.step % o.eval_every == 0:
                res.eval_losses.append((self.step, self.evaluate(eval_batches)))
            if out_dir and o.save_every and self.step % o.save_every == 0:
                self.save_checkpoint(os.path.join(out_dir, f"checkpoint-{self.step}"))
        if eval_batches:
            res.eval_losses.append((self.step, self.evaluate(eval_batches)))
        if out_dir and self._is_writer():
            os.makedirs(out_dir, exist_ok=True)
            save_adapters(self.model, out_dir)
            with open(os.path.join(out_dir, "finetuning.json"), "w") as f:
                json.dump({"options": asdict(o), "steps": res.steps, "tokens": res.tokens,
                           "final_loss": res.losses[-1] if res.losses else None, "eval": res.eval_losses}, f, indent=1)
            res.adapter_folder = out_dir
        return res

    def _is_writer(self) -> bool:
        return not dist.is_initialized() or dist.get_rank(self.group) == 0

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, folder: str) -> None:
        # the sharded optimizer's state is gathered by all ranks (one file whatever the world size), then one writes
        state = self.sync.optimizer_state() if self.sync is not None else None
        if not self._is_writer():
            return
        os.makedirs(folder, exist_ok=True)
        save_adapters(self.model, folder)
        from ..formats.safetensors import save_file
        if state is None:
            state = self.optimizer.state_dict()
        save_file({k: v for k, v in state.items() if isinstance(v, torch.Tensor)},
                  os.path.join(folder, "optimizer.safetensors"), metadata={"format": "idrak-optimizer", "optimizer": "AdamW"})
        with open(os.path.join(folder, "train-state.json"), "w") as f:
            json.dump({"step": self.step, "tokens": self.result.tokens, "losses": self.result.losses[-16:]}, f)

    def load_checkpoint(self, folder: str) -> None:
        """Optimizer moments and the step counter of a checkpoint whose adapters are already attached."""
        from ..formats.safetensors import load_file
        path = os.path.join(folder, "optimizer.safetensors")
        if os.path.isfile(path):
            if self.sync is not None:
                self.sync.load_optimizer_state(load_file(path))
            else:
                self.optimizer.load_state_dict(load_file(path))
        with open(os.path.join(folder, "train-state.json")) as f:
            st = json.load(f)
        self.step, self.result.tokens = int(st["step"]), int(st.get("tokens", 0))

    # ------------------------------------------------------------------ one call
    @staticmethod
    def train(model, tokenizer, train: Sequence[Dict[str, Any]], evaluation=None,
              options: Optional[FineTuningOptions] = None, out_dir: Optional[str] = None, progress=None,
              group=None) -> FineTuningResult:
        return FineTuner(model, tokenizer, options, group).fit(train, evaluation, out_dir, progress)
