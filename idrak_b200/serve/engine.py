"""Continuous-batching generation engine over token ids.

``LLMEngine`` owns a model runner (paged KV cache + kernels) and the native scheduler. ``add_request`` queues a
prompt; every ``step`` runs either one packed prefill of newly admitted prompts or one decode token for all
running sequences, samples on the device, and returns the new tokens. ``generate`` drives steps until the given
prompts finish. Requests come and go between steps - a late request joins the running batch at its next step
instead of waiting for the batch to drain.

Reference: GenerationOptions defaults (src/Idrak.Abstraction/Generation/GenerationOptions.cs:14-181), TextGenerator
Generate / GenerateBatch (src/Idrak/Generation/TextGenerator.cs:38), device-side sampling with one host read per
chunk (src/Idrak.Gpu/Cuda/PtxKernels.Decoding.cs:12).
"""
from __future__ import annotations

import itertools
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..models.decoder import Decoder
from ..ops import decode as dops
from .runner import ModelRunner, PrefillItem
from .scheduler import DECODE, PREFILL, QueueFull, Scheduler


@dataclass
class GenerationOptions:
    """Sampling and stopping settings of one request (defaults follow the reference's GenerationOptions)."""
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    repeat_penalty: float = 1.1
    repeat_last_n: int = 64
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    max_tokens: int = 128                       # NumPredict; <= 0 means "until the context is full"
    stop_token_ids: Tuple[int, ...] = ()
    stop: Tuple[str, ...] = ()                  # stop strings: applied by the text layer
    return_logprobs: bool = False
    repeat_stop: bool = False                   # stop when the tail repeats itself (RepeatStop)
    repeat_stop_min_tokens: int = 4
    timeout: float = 0.0                        # seconds a request may wait in the queue (0 = forever)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def penalised(self) -> bool:
        return self.repeat_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @staticmethod
    def greedy_options(max_tokens: int = 128, **kw) -> "GenerationOptions":
        return GenerationOptions(temperature=0.0, top_k=1, top_p=1.0, repeat_penalty=1.0, max_tokens=max_tokens, **kw)


@dataclass
class StepOutput:
    request_id: int
    token: int                   # -1 when the request ended without a new token (expired / aborted)
    finished: bool
    finish_reason: Optional[str] = None       # "stop" | "length" | "timeout" | "abort" | "repeat"
    logprob: Optional[float] = None


@dataclass
class Request:
    id: int
    prompt: List[int]
    options: GenerationOptions
    output: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    arrival: float = 0.0
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    seed: int = 0
    on_token: Optional[Callable[[StepOutput], None]] = None
    blocks: List[int] = field(default_factory=list)


def _tail_repeats(tokens: Sequence[int], min_tokens: int) -> bool:
    """True when the last ``p`` tokens repeat the ``p`` before them three times over, for some p >= min_tokens / 2."""
    n = len(tokens)
    for p in range(max(min_tokens // 2, 1), 65):
        if n < 3 * p:
            break
        if tokens[n - p:] == tokens[n - 2 * p: n - p] == tokens[n - 3 * p: n - 2 * p]:
            return True
    return False


class LLMEngine:
    def __init__(self, model: Decoder, num_blocks: Optional[int] = None, block_size: int = 16, max_batch: int = 64,
                 max_prefill_tokens: int = 8192, queue_limit: int = 0, prefix_sharing: bool = True,
                 eos_token_ids: Sequence[int] = (), cache_bytes: Optional[int] = None,
                 clock: Callable[[], float] = time.monotonic, use_graph: bool = True, tp=None,
                 kv_dtype: Optional[torch.dtype] = None, fold_norms: bool = False):
        """``fold_norms``: rewrite the model (in place, inference only) so that each RMS norm's weight is multiplied into
        the projection that follows it; decode steps of up to 64 sequences then run the norm inside the projection
        kernels (``serve.runner.fold_norms_into_projections``).

        ``tp``: a ``parallel.tp_serve.TPServeContext`` when ``model`` is one rank's slice of a tensor-parallel
        decoder. Every rank of the group then runs an engine of its own over the same requests in lock-step: the
        scheduler is deterministic and the sampled tokens are equal on every rank, so the engines stay in step
        without exchanging anything but the activations."""
        spec = model.spec
        p = next(model.parameters())
        if num_blocks is None:
            if cache_bytes is None:
                if p.is_cuda:
                    free, _ = torch.cuda.mem_get_info(p.device)
                    cache_bytes = int(free * 0.8)
                else:
                    cache_bytes = 256 << 20
            num_blocks = ModelRunner.blocks_that_fit(spec, cache_bytes, block_size,
                                                     1 if kv_dtype == torch.int8 else p.element_size())
            # no point in holding more than every slot at full context
            num_blocks = min(num_blocks, max_batch * ((spec.max_positions + block_size - 1) // block_size))
            if tp is not None:
                # the ranks' schedulers must make the same decisions: size every cache like the smallest
                import torch.distributed as dist
                t = torch.tensor([num_blocks], dtype=torch.int64, device=p.device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=tp.comm.group)
                num_blocks = int(t.item())
        self.spec, self.block_size = spec, block_size
        self.tp = tp
        if tp is not None:
            from .tp_runner import TPModelRunner
            self.runner = TPModelRunner(model, num_blocks, block_size, max_batch, kv_dtype, tp=tp)
            self.spec = spec = model.tp_full_spec       # token ids, end-of-sequence checks and limits are the whole model's
        else:
            if fold_norms:
                from .runner import fold_norms_into_projections
                fold_norms_into_projections(model)
            self.runner = ModelRunner(model, num_blocks, block_size, max_batch, kv_dtype)
        self.sched = Scheduler(num_blocks, block_size, max_batch, max_prefill_tokens, queue_limit, prefix_sharing)
        self.eos = set(int(t) for t in eos_token_ids)
        self.clock = clock
        self.requests: Dict[int, Request] = {}
        self._ids = itertools.count(1)
        self._lock = threading.RLock()
        self.device = self.runner.device
        self.tokens_generated = 0
        self.tokens_prefilled = 0
        self.steps = 0
        self.phase_seconds = {"prefill": 0.0, "decode": 0.0}
        self.phase_steps = {"prefill": 0, "decode": 0}
        self.use_graph = bool(use_graph) and self.device.type == "cuda"
        self.last_error: Optional[BaseException] = None

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], options: Optional[GenerationOptions] = None,
                    on_token: Optional[Callable[[StepOutput], None]] = None) -> int:
        options = options or GenerationOptions()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        limit = self.spec.max_positions
        if len(prompt) >= limit:
            raise ValueError(f"the prompt has {len(prompt)} tokens; the model's context holds {limit}")
        room = limit - len(prompt)
        max_new = options.max_tokens if options.max_tokens > 0 else room
        max_new = min(max_new, room)
        with self._lock:
            rid = next(self._ids)
            now = self.clock()
            deadline = now + options.timeout if options.timeout > 0 else 0.0
            self.sched.add(rid, prompt, max_new, deadline)
            seed = options.seed if options.seed is not None else (0x9E3779B97F4A7C15 * rid) & 0x7FFFFFFFFFFFFFFF
            self.requests[rid] = Request(rid, prompt, options, arrival=now, seed=seed, on_token=on_token)
            return rid

    def abort(self, request_id: int) -> None:
        with self._lock:
            r = self.requests.get(request_id)
            if r is None or r.finished:
                return
            self.sched.abort(request_id)
            self._finish(r, "abort")
            if r.on_token:
                r.on_token(StepOutput(r.id, -1, True, "abort"))

    def fail_all(self, error: BaseException) -> None:
        """End every unfinished request with reason "error" (a step raised): callers waiting on them wake up."""
        with self._lock:
            self.last_error = error
            for r in list(self.requests.values()):
                if not r.finished:
                    self.sched.abort(r.id)
                    self._finish(r, "error")
                    if r.on_token:
                        r.on_token(StepOutput(r.id, -1, True, "error"))

    def release(self, request_id: int) -> Optional[Request]:
        """Forget a finished request (its record is returned)."""
        with self._lock:
            r = self.requests.pop(request_id, None)
            self.sched.forget(request_id)
            return r

    def has_work(self) -> bool:
        st = self.sched.stats()
        return st["waiting"] + st["running"] > 0

    def _finish(self, r: Request, reason: str) -> None:
        r.finished, r.finish_reason, r.finished_at = True, reason, self.clock()

    # ------------------------------------------------------------------ sampling
    def _sample(self, logits: torch.Tensor, reqs: List[Request]) -> Tuple[List[int], Optional[List[float]]]:
        """Pick one token per row on the device; one host read of ``len(reqs)`` ints."""
        vocab, dev = self.spec.vocabulary, logits.device
        want_lp = any(r.options.return_logprobs for r in reqs)
        all_greedy = all(r.options.greedy and not r.options.penalised for r in reqs)
        if self.tp is not None:
            if all_greedy and not want_lp:
                # per-rank arg-max of the vocabulary slice, merged across ranks on the device
                ids = self.tp.argmax(logits, self.runner.vocab_local, self.runner.vocab_offset)
                return ids.tolist(), None
            logits = self.tp.gather_logits(logits)      # the whole distribution for samplers that need it
        if all_greedy:
            ids = dops.argmax_rows(logits, vocab)
        else:
            o = [r.options for r in reqs]
            f32 = lambda xs: torch.tensor(xs, dtype=torch.float32, device=dev)
            temperature = f32([1.0 if x.greedy else x.temperature for x in o])
            top_k = torch.tensor([1 if x.greedy else x.top_k for x in o], dtype=torch.int32, device=dev)
            top_p, min_p = f32([x.top_p for x in o]), f32([x.min_p for x in o])
            # a request's draws depend on its seed and its own token index only, not on its batch neighbours
            seeds = torch.tensor([(r.seed + 0x9E3779B97F4A7C15 * (len(r.output) + 1)) & 0x7FFFFFFFFFFFFFFF
                                  for r in reqs], dtype=torch.int64, device=dev)
            history = rp = pp = fp = None
            if any(x.penalised for x in o):
                width = max(max(x.repeat_last_n for x in o), 1)
                rows = []
                for r in reqs:
                    n = r.options.repeat_last_n if r.options.penalised else 0
                    tail = (r.prompt + r.output)[-n:] if n > 0 else []
                    rows.append(tail + [-1] * (width - len(tail)))
                history = torch.tensor(rows, dtype=torch.int32, device=dev)
                rp, pp, fp = (f32([x.repeat_penalty for x in o]), f32([x.presence_penalty for x in o]),
                              f32([x.frequency_penalty for x in o]))
            ids = dops.sample_rows(logits, vocab, temperature, top_k, top_p, min_p, seeds, 0,
                                   history, rp, pp, fp)
        lps = None
        if want_lp:
            lp = torch.log_softmax(logits[:, :vocab].float(), -1)
            lps = lp.gather(1, ids.long()[:, None])[:, 0].tolist()
        return ids.tolist(), lps

    # ------------------------------------------------------------------ one step
    def step(self) -> List[StepOutput]:
        with self._lock:
            return self._step()

    def _step(self) -> List[StepOutput]:
        now = self.clock()
        kind, ids, expired = self.sched.step(now)
        outs: List[StepOutput] = []
        for rid in expired:
            r = self.requests.get(rid)
            if r is not None and not r.finished:
                self._finish(r, "timeout")
                outs.append(StepOutput(rid, -1, True, "timeout"))
        if not ids:
            self._notify(outs)
            return outs
        self.steps += 1
        started = time.perf_counter()
        reqs = [self.requests[i] for i in ids]
        bs = self.block_size
        if kind == PREFILL:
            items = []
            for r in reqs:
                info = self.sched.info(r.id)
                toks = self.sched.tokens(r.id, info.length)
                r.blocks = self.sched.blocks(r.id, info.n_blocks)
                items.append(PrefillItem(toks[info.cached_prefix:], info.cached_prefix, r.blocks))
                self.tokens_prefilled += info.length - info.cached_prefix
            logits = self.runner.prefill(items)
        else:
            n = len(reqs)
            longest = 0
            for r in reqs:
                length = len(r.prompt) + len(r.output)
                need = (length + bs - 1) // bs
                if len(r.blocks) < need:
                    r.blocks = self.sched.blocks(r.id, self.sched.info(r.id).n_blocks)
                longest = max(longest, length)
            width = max(len(r.blocks) for r in reqs)
            table = torch.tensor([r.blocks + [0] * (width - len(r.blocks)) for r in reqs], dtype=torch.int32)
            last = torch.tensor([(r.output[-1] if r.output else r.prompt[-1]) for r in reqs], dtype=torch.int32)
            pos = torch.tensor([len(r.prompt) + len(r.output) - 1 for r in reqs], dtype=torch.int32)
            dev = self.device
            if dev.type == "cuda":
                table, last, pos = (t.pin_memory().to(dev, non_blocking=True) for t in (table, last, pos))
            if self.use_graph:
                logits = self.runner.decode_graphed(last, pos, table, longest)
            else:
                logits = self.runner.decode(last, pos, table, max_len_hint=longest)
        tokens, lps = self._sample(logits, reqs)       # reads the tokens back: the step's device work is done here
        phase = "prefill" if kind == PREFILL else "decode"
        self.phase_seconds[phase] += time.perf_counter() - started
        self.phase_steps[phase] += 1
        now = self.clock()
        for i, r in enumerate(reqs):
            tok = int(tokens[i])
            r.output.append(tok)
            if lps is not None:
                r.logprobs.append(float(lps[i]))
            if r.first_token_at is None:
                r.first_token_at = now
            self.tokens_generated += 1
            reason = None
            if tok in self.eos or tok in r.options.stop_token_ids:
                reason = "stop"
            elif r.options.repeat_stop and _tail_repeats(r.output, r.options.repeat_stop_min_tokens):
                reason = "repeat"
            done = self.sched.commit(r.id, tok, reason is not None)
            if done and reason is None:
                reason = "length"
            if done:
                self._finish(r, reason)
            outs.append(StepOutput(r.id, tok, done, reason, lps[i] if lps is not None else None))
        self._notify(outs)
        return outs

    def _notify(self, outs: List[StepOutput]) -> None:
        for o in outs:
            r = self.requests.get(o.request_id)
            if r is not None and r.on_token is not None:
                r.on_token(o)

    # ------------------------------------------------------------------ batch convenience
    def generate(self, prompts: Sequence[Sequence[int]], options=None) -> List[Request]:
        """Run the prompts to completion (continuous batching between them) and return their records in order.
        A stop / end-of-sequence token ends a request and is kept as its last output token."""
        if options is None or isinstance(options, GenerationOptions):
            options = [options] * len(prompts)
        ids = [self.add_request(p, o) for p, o in zip(prompts, options)]
        while any(not self.requests[i].finished for i in ids):
            if not self.step() and not self.has_work():
                break
        return [self.release(i) for i in ids]

    def stats(self) -> dict:
        s = self.sched.stats()
        s.update(tokens_generated=self.tokens_generated, tokens_prefilled=self.tokens_prefilled, steps=self.steps,
                 prefill_seconds=self.phase_seconds["prefill"], decode_seconds=self.phase_seconds["decode"],
                 prefill_steps=self.phase_steps["prefill"], decode_steps=self.phase_steps["decode"])
        return s
