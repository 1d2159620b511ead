"""Text in, text out: tokenise, run the continuous-batching engine, detokenise while streaming, honour stop strings.

``TextGenerator`` serves any number of concurrent callers from one engine. Without a background loop the calling
thread drives the engine's steps itself; with ``start()`` a loop thread steps the engine and callers only wait on
their own token queues, which is how the HTTP server uses it. Conversation turns reuse the KV blocks of their
common prefix through the scheduler's prefix sharing.

Reference: TextGenerator Generate / Stream / GenerateBatch / StreamBatch, stop strings, repeat-loop stop, returned
tokens and log-probabilities (src/Idrak/Generation/TextGenerator.cs:38,569-623).
"""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Sequence, Union

from ..serve.engine import GenerationOptions, LLMEngine, StepOutput
from ..text.chat import ChatTemplate
from ..text.tokenizer import Tokenizer
from ..text.tool_calls import ToolCall, _held_suffix


@dataclass
class GenerationResult:
    text: str = ""
    tokens: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    finish_reason: Optional[str] = None          # stop | length | timeout | abort | repeat
    prompt_tokens: int = 0
    tool_calls: List[ToolCall] = field(default_factory=list)
    queue_seconds: float = 0.0
    total_seconds: float = 0.0

    @property
    def completion_tokens(self) -> int:
        return len(self.tokens)


class _StopFilter:
    """Passes text through, holding back what may become a stop string; reports when one is complete."""

    def __init__(self, stops: Sequence[str]):
        self.stops = [s for s in stops if s]
        self.buf = ""
        self.hit = False

    def push(self, piece: str) -> str:
        if self.hit:
            return ""
        self.buf += piece
        first = min((i for i in (self.buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if first >= 0:
            out, self.buf, self.hit = self.buf[:first], "", True
            return out
        hold = max((_held_suffix(self.buf, s) for s in self.stops), default=0)
        out, self.buf = self.buf[: len(self.buf) - hold], self.buf[len(self.buf) - hold:]
        return out

    def flush(self) -> str:
        out, self.buf = ("" if self.hit else self.buf), ""
        return out


class TextGenerator:
    def __init__(self, model=None, tokenizer: Tokenizer = None, engine: Optional[LLMEngine] = None, **engine_args):
        if tokenizer is None:
            raise ValueError("a tokenizer is required")
        self.tokenizer = tokenizer
        if engine is None:
            engine_args.setdefault("eos_token_ids", tuple(tokenizer.eos_token_ids))
            engine = LLMEngine(model, **engine_args)
        self.engine = engine
        self.template = ChatTemplate.for_tokenizer(tokenizer)
        self._thread: Optional[threading.Thread] = None
        self._wake = threading.Event()
        self._stopping = False

    # ------------------------------------------------------------------ background loop
    def start(self) -> "TextGenerator":
        if self._thread is None:
            self._stopping = False
            self._thread = threading.Thread(target=self._loop, name="idrak-engine", daemon=True)
            self._thread.start()
        return self

    def close(self) -> None:
        self._stopping = True
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=30)
            self._thread = None

    def _loop(self) -> None:
        dev = self.engine.device
        if dev.type == "cuda":
            import torch
            torch.cuda.set_device(dev)
        while not self._stopping:
            if self.engine.has_work():
                try:
                    self.engine.step()
                except Exception as e:        # a failed step must not strand the callers waiting on their queues
                    self.engine.fail_all(e)
            else:
                self._wake.wait(0.05)
                self._wake.clear()

    # ------------------------------------------------------------------ prompts
    def encode_prompt(self, prompt: Union[str, Sequence[int], Sequence[Dict[str, Any]]], tools=None) -> List[int]:
        if isinstance(prompt, str):
            return self.tokenizer.encode(prompt, add_special_tokens=True)
        prompt = list(prompt)
        if prompt and isinstance(prompt[0], dict):
            text = self.template.render(prompt, tools=tools, add_generation_prompt=True)
            return self.tokenizer.encode(text, add_special_tokens=False)
        return [int(t) for t in prompt]

    # ------------------------------------------------------------------ streaming core
    def _submit(self, prompt, options, tools, res: GenerationResult) -> "_Pending":
        options = options or GenerationOptions()
        ids = self.encode_prompt(prompt, tools)
        res.prompt_tokens = len(ids)
        q: "queue.Queue[StepOutput]" = queue.Queue()
        rid = self.engine.add_request(ids, options, on_token=q.put)
        self._wake.set()
        return _Pending(rid, q, options, res, self.tokenizer.stream(skip_special_tokens=True),
                        _StopFilter(options.stop), set(self.engine.eos) | set(options.stop_token_ids))

    def _consume(self, p: "_Pending") -> Iterator[str]:
        res, stops, decoder, q = p.result, p.stops, p.decoder, p.queue
        try:
            done = False
            while not done:
                if self._thread is None:
                    while q.empty():
                        if not self.engine.step() and not self.engine.has_work() and q.empty():
                            raise RuntimeError("the engine has no work left but the request has not finished")
                out = q.get()
                if out.token >= 0:
                    res.tokens.append(out.token)
                    if out.logprob is not None:
                        res.logprobs.append(out.logprob)
                    if not (out.finished and out.token in p.stop_ids):
                        piece = stops.push(decoder.push(out.token))
                        if piece:
                            res.text += piece
                            yield piece
                if stops.hit and not out.finished:
                    self.engine.abort(p.request_id)
                    res.finish_reason = "stop"
                    break
                if out.finished:
                    done = True
                    res.finish_reason = "stop" if stops.hit else out.finish_reason
                    if out.finish_reason == "error":
                        raise RuntimeError(f"generation failed: {self.engine.last_error!r}") from self.engine.last_error
            if not stops.hit:
                tail = stops.push(decoder.flush()) + stops.flush()
                if tail:
                    res.text += tail
                    yield tail
        finally:
            r = self.engine.requests.get(p.request_id)
            if r is not None and not r.finished:
                self.engine.abort(p.request_id)
            r = self.engine.release(p.request_id)
            if r is not None:
                res.queue_seconds = (r.first_token_at or r.finished_at or r.arrival) - r.arrival
                res.total_seconds = (r.finished_at or r.arrival) - r.arrival

    def stream_events(self, prompt, options: Optional[GenerationOptions] = None, tools=None,
                      result: Optional[GenerationResult] = None) -> Iterator[str]:
        """Yield text pieces as they are produced; fills ``result`` (text, tokens, finish reason, timings).
        The request joins the engine at the call, not at the first ``next()``."""
        res = result if result is not None else GenerationResult()
        return self._consume(self._submit(prompt, options, tools, res))

    # ------------------------------------------------------------------ public calls
    def stream(self, prompt, options: Optional[GenerationOptions] = None, tools=None) -> Iterator[str]:
        return self.stream_events(prompt, options, tools)

    def generate(self, prompt, options: Optional[GenerationOptions] = None, tools=None) -> GenerationResult:
        res = GenerationResult()
        for _ in self.stream_events(prompt, options, tools, res):
            pass
        if tools and isinstance(prompt, (list, tuple)) and prompt and isinstance(prompt[0], dict):
            parser = self.template.parser(tools)
            a, b = parser.feed(res.text), parser.finish()
            res.tool_calls = a.tool_calls + b.tool_calls
            if res.tool_calls:
                res.text = a.content + b.content
                res.finish_reason = "tool_calls" if res.finish_reason == "stop" else res.finish_reason
        return res

    def chat(self, messages: Sequence[Dict[str, Any]], options: Optional[GenerationOptions] = None,
             tools: Optional[List[dict]] = None) -> GenerationResult:
        return self.generate(list(messages), options, tools)

    def generate_batch(self, prompts: Sequence, options=None) -> List[GenerationResult]:
        """All prompts join the engine first and run together (continuous batching); results come back in order."""
        if options is None or isinstance(options, GenerationOptions):
            options = [options] * len(prompts)
        results = [GenerationResult() for _ in prompts]
        streams = [self.stream_events(p, o, None, r) for p, o, r in zip(prompts, options, results)]
        for s in streams:         # the first stream's waits drive the engine for all; later ones find tokens queued
            for _ in s:
                pass
        return results

    def stream_batch(self, prompts: Sequence, options=None) -> Iterator[tuple]:
        """Yield ``(index, piece)`` as pieces of any prompt arrive."""
        if options is None or isinstance(options, GenerationOptions):
            options = [options] * len(prompts)
        streams = [self.stream_events(p, o) for p, o in zip(prompts, options)]
        live = dict(enumerate(streams))
        while live:
            for i in list(live):
                try:
                    yield i, next(live[i])
                except StopIteration:
                    del live[i]


@dataclass
class _Pending:
    request_id: int
    queue: "queue.Queue[StepOutput]"
    options: GenerationOptions
    result: GenerationResult
    decoder: Any
    stops: _StopFilter
    stop_ids: set
