"""Named models behind one engine: load on first use, copies, leases, queue limits, timeouts, keep-alive, stats.

    engine = (InferenceEngine.create()
              .add_chat("assistant", load=lambda: (model, tokenizer), queue_limit=64, keep_alive=300)
              .add_predictor("scorer", load=lambda: torch_module, copies=2, micro_batch=16)
              .build())
    engine.chat("assistant", messages)            # text / chat models: continuous batching inside one copy
    engine.predict("scorer", tensor)              # predictors: round-robin copies or exclusive leases

Reference: InferenceEngine builder, HostedModel (copies, leases, queue limit -> InferenceQueueFullException, timeout,
keep-alive unload, micro-batcher), EngineStats (src/Idrak/Inference/*, src/Idrak.Abstraction/Serving/EngineModel.cs:181-200).
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence

from .engine import GenerationOptions
from .scheduler import QueueFull


class InferenceQueueFull(RuntimeError):
    """More requests are waiting for the model than its queue limit allows."""


class InferenceTimeout(TimeoutError):
    """The request waited longer than the model's timeout for a free copy."""


class EngineStats:
    """Request counts and latency summary of one hosted model (rolling window of the last 1,024 requests)."""

    def __init__(self):
        self._lock = threading.Lock()
        self.requests = self.failures = self.rejected = self.timeouts = 0
        self.loads = self.unloads = 0
        self._latency: deque = deque(maxlen=1024)
        self._wait: deque = deque(maxlen=1024)

    def record(self, latency: float, wait: float, ok: bool = True) -> None:
        with self._lock:
            self.requests += 1
            self.failures += 0 if ok else 1
            self._latency.append(latency)
            self._wait.append(wait)

    @staticmethod
    def _p95(values) -> float:
        if not values:
            return 0.0
        v = sorted(values)
        return v[min(len(v) - 1, int(0.95 * len(v)))]

    def snapshot(self) -> dict:
        with self._lock:
            lat, wait = list(self._latency), list(self._wait)
            return {"requests": self.requests, "failures": self.failures, "rejected": self.rejected,
                    "timeouts": self.timeouts, "loads": self.loads, "unloads": self.unloads,
                    "average_latency": sum(lat) / len(lat) if lat else 0.0, "p95_latency": self._p95(lat),
                    "average_queue_wait": sum(wait) / len(wait) if wait else 0.0, "p95_queue_wait": self._p95(wait)}


@dataclass
class ModelSettings:
    name: str
    kind: str                                   # predictor | text | chat | embed | a registered plug-in kind
    load: Callable[[], Any]
    copies: int = 1
    exclusive: bool = False                     # a caller holds a copy alone for the duration of its call
    queue_limit: int = 0                        # 0 = unbounded
    timeout: float = 0.0                        # seconds to wait for a copy (0 = forever)
    keep_alive: float = 0.0                     # seconds idle before the copies are unloaded (0 = never)
    micro_batch: int = 0                        # predictors: gather up to this many calls into one forward
    micro_batch_wait: float = 0.002
    engine_args: Dict[str, Any] = field(default_factory=dict)
    description: str = ""


class HostedModel:
    def __init__(self, settings: ModelSettings, clock: Callable[[], float] = time.monotonic):
        self.settings, self.clock = settings, clock
        self.stats = EngineStats()
        self._lock = threading.Condition()
        self._copies: List[Any] = []
        self._busy: List[bool] = []
        self._next = 0
        self._waiting = 0
        self._active = 0
        self._last_used = clock()
        self._batcher: Optional[_MicroBatcher] = None
        self.loaded_at: Optional[float] = None

    # ------------------------------------------------------------------ lifetime
    @property
    def loaded(self) -> bool:
        return bool(self._copies)

    def _ensure_loaded(self) -> None:
        if self._copies:
            return
        s = self.settings
        made = [self._wrap(s.load()) for _ in range(max(s.copies, 1))]
        self._copies, self._busy = made, [False] * len(made)
        self.loaded_at = self.clock()
        self.stats.loads += 1
        if s.kind == "predictor" and s.micro_batch > 1:
            self._batcher = _MicroBatcher(self, s.micro_batch, s.micro_batch_wait)

    def _wrap(self, loaded: Any) -> Any:
        s = self.settings
        if s.kind in ("text", "chat", "embed"):
            from ..generation.text_generator import TextGenerator
            if isinstance(loaded, TextGenerator):
                return loaded.start()
            model, tokenizer = loaded
            args = dict(s.engine_args)
            args.setdefault("queue_limit", s.queue_limit)
            return TextGenerator(model, tokenizer, **args).start()
        return loaded

    def unload(self) -> bool:
        with self._lock:
            if not self._copies or self._active > 0:
                return False
            for c in self._copies:
                close = getattr(c, "close", None)
                if callable(close):
                    close()
            if self._batcher is not None:
                self._batcher.close()
                self._batcher = None
            self._copies, self._busy, self.loaded_at = [], [], None
            self.stats.unloads += 1
            return True

    def expire_if_idle(self) -> bool:
        s = self.settings
        if s.keep_alive > 0 and self._copies and self._active == 0 and self.clock() - self._last_used >= s.keep_alive:
            return self.unload()
        return False

    # ------------------------------------------------------------------ leases
    def acquire(self):
        """A copy for one call: shared copies go round-robin; exclusive ones are waited for (queue limit, timeout)."""
        s = self.settings
        start = self.clock()
        with self._lock:
            self._ensure_loaded()
            if not s.exclusive:
                i = self._next % len(self._copies)
                self._next += 1
                self._active += 1
                return i, self._copies[i], 0.0
            if s.queue_limit > 0 and self._waiting >= s.queue_limit and all(self._busy):
                self.stats.rejected += 1
                raise InferenceQueueFull(f"model '{s.name}': {self._waiting} requests are already waiting "
                                         f"(queue limit {s.queue_limit})")
            self._waiting += 1
            try:
                while all(self._busy):
                    left = None if s.timeout <= 0 else s.timeout - (self.clock() - start)
                    if left is not None and left <= 0:
                        self.stats.timeouts += 1
                        raise InferenceTimeout(f"model '{s.name}': no copy became free within {s.timeout:g} s")
                    self._lock.wait(left)
            finally:
                self._waiting -= 1
            i = self._busy.index(False)
            self._busy[i] = True
            self._active += 1
            return i, self._copies[i], self.clock() - start

    def release(self, index: int) -> None:
        with self._lock:
            if self.settings.exclusive and index < len(self._busy):
                self._busy[index] = False
            self._active -= 1
            self._last_used = self.clock()
            self._lock.notify()

    def run(self, fn: Callable[[Any], Any]) -> Any:
        start = self.clock()
        i, copy, waited = self.acquire()
        ok = False
        try:
            out = fn(copy)
            ok = True
            return out
        finally:
            self.release(i)
            self.stats.record(self.clock() - start, waited, ok)

    def status(self) -> dict:
        s = self.settings
        return {"name": s.name, "kind": s.kind, "loaded": self.loaded, "copies": s.copies, "active": self._active,
                "waiting": self._waiting, "keep_alive": s.keep_alive, "description": s.description,
                "expires_in": (max(0.0, s.keep_alive - (self.clock() - self._last_used))
                               if s.keep_alive > 0 and self.loaded and self._active == 0 else None),
                **self.stats.snapshot()}


class _MicroBatcher:
    """Gathers predictor calls that arrive within a short window into one batched forward on a worker thread."""

    def __init__(self, host: HostedModel, limit: int, wait: float):
        self.host, self.limit, self.wait = host, limit, wait
        self._items: List[tuple] = []
        self._cv = threading.Condition()
        self._closing = False
        self.batches = 0
        self._thread = threading.Thread(target=self._loop, name=f"idrak-batch-{host.settings.name}", daemon=True)
        self._thread.start()

    def submit(self, x):
        done = threading.Event()
        slot = [None, None]
        with self._cv:
            self._items.append((x, slot, done))
            self._cv.notify()
        done.wait()
        if slot[1] is not None:
            raise slot[1]
        return slot[0]

    def close(self):
        with self._cv:
            self._closing = True
            self._cv.notify()
        self._thread.join(timeout=10)

    def _loop(self):
        import torch
        while True:
            with self._cv:
                while not self._items and not self._closing:
                    self._cv.wait()
                if self._closing and not self._items:
                    return
                deadline = time.monotonic() + self.wait
                while len(self._items) < self.limit:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        break
                    self._cv.wait(left)
                batch, self._items = self._items[: self.limit], self._items[self.limit:]
            try:
                xs = torch.stack([b[0] for b in batch])
                ys = self.host.run(lambda m: m(xs))
                self.batches += 1
                for (_, slot, done), y in zip(batch, ys):
                    slot[0] = y
                    done.set()
            except Exception as e:           # every caller of the batch sees the failure
                for _, slot, done in batch:
                    slot[1] = e
                    done.set()


_PLUGIN_KINDS: Dict[str, Callable[[Any, Any], Any]] = {}


def register_model_kind(kind: str, call: Callable[[Any, Any], Any]) -> None:
    """A plug-in model kind: ``call(loaded_copy, request) -> response`` serves ``InferenceEngine.invoke``."""
    _PLUGIN_KINDS[kind] = call


class InferenceEngineBuilder:
    def __init__(self):
        self._models: List[ModelSettings] = []
        self._clock = time.monotonic

    def _add(self, kind, name, load, **kw) -> "InferenceEngineBuilder":
        if any(m.name == name for m in self._models):
            raise ValueError(f"a model named '{name}' is already registered")
        self._models.append(ModelSettings(name=name, kind=kind, load=load, **kw))
        return self

    def add_predictor(self, name, load, **kw):
        return self._add("predictor", name, load, **kw)

    def add_text(self, name, load, **kw):
        return self._add("text", name, load, **kw)

    def add_chat(self, name, load, **kw):
        return self._add("chat", name, load, **kw)

    def add_embed(self, name, load, **kw):
        return self._add("embed", name, load, **kw)

    def add_plugin(self, kind, name, load, **kw):
        if kind not in _PLUGIN_KINDS:
            raise KeyError(f"model kind '{kind}' is not registered: add it with register_model_kind")
        return self._add(kind, name, load, **kw)

    def with_clock(self, clock):
        self._clock = clock
        return self

    def build(self, preload: Sequence[str] = ()) -> "InferenceEngine":
        eng = InferenceEngine([HostedModel(m, self._clock) for m in self._models])
        for name in preload:
            with eng.model(name)._lock:
                eng.model(name)._ensure_loaded()
        return eng


class InferenceEngine:
    def __init__(self, hosted: Sequence[HostedModel]):
        self._models = {h.settings.name: h for h in hosted}
        self._stop = threading.Event()
        self._reaper: Optional[threading.Thread] = None
        if any(h.settings.keep_alive > 0 for h in hosted):
            self._reaper = threading.Thread(target=self._reap, name="idrak-keep-alive", daemon=True)
            self._reaper.start()

    @staticmethod
    def create() -> InferenceEngineBuilder:
        return InferenceEngineBuilder()

    def _reap(self):
        while not self._stop.wait(0.25):
            self.expire_idle()

    def expire_idle(self) -> List[str]:
        return [n for n, h in self._models.items() if h.expire_if_idle()]

    def close(self):
        self._stop.set()
        for h in self._models.values():
            h.unload()

    # ------------------------------------------------------------------ look-up
    def model(self, name: str) -> HostedModel:
        if name not in self._models:
            raise KeyError(f"no model named '{name}'. Known: {', '.join(sorted(self._models)) or '(none)'}")
        return self._models[name]

    def names(self, kind: Optional[str] = None) -> List[str]:
        return [n for n, h in self._models.items() if kind is None or h.settings.kind == kind]

    def statuses(self) -> List[dict]:
        return [h.status() for h in self._models.values()]

    def _of_kind(self, name, kinds) -> HostedModel:
        h = self.model(name)
        if h.settings.kind not in kinds:
            raise TypeError(f"model '{name}' is a {h.settings.kind} model; this call needs {' or '.join(kinds)}")
        return h

    # ------------------------------------------------------------------ calls
    def predict(self, name: str, x):
        h = self._of_kind(name, ("predictor",))
        with h._lock:
            h._ensure_loaded()
        if h._batcher is not None:
            return h._batcher.submit(x)
        return h.run(lambda m: m(x))

    def _options(self, h: HostedModel, options: Optional[GenerationOptions]) -> GenerationOptions:
        import dataclasses
        o = options or GenerationOptions()
        if h.settings.timeout > 0 and o.timeout <= 0:
            o = dataclasses.replace(o, timeout=h.settings.timeout)
        return o

    def _text_call(self, h: HostedModel, fn):
        try:
            out = h.run(fn)
        except QueueFull as e:
            h.stats.rejected += 1
            raise InferenceQueueFull(f"model '{h.settings.name}': {e}") from e
        if getattr(out, "finish_reason", None) == "timeout":
            h.stats.timeouts += 1
            raise InferenceTimeout(f"model '{h.settings.name}': the request waited longer than its timeout in the queue")
        return out

    def generate(self, name: str, prompt, options: Optional[GenerationOptions] = None):
        h = self._of_kind(name, ("text", "chat"))
        o = self._options(h, options)
        return self._text_call(h, lambda g: g.generate(prompt, o))

    def chat(self, name: str, messages, options: Optional[GenerationOptions] = None, tools=None):
        h = self._of_kind(name, ("chat",))
        o = self._options(h, options)
        return self._text_call(h, lambda g: g.chat(messages, o, tools))

    def stream(self, name: str, prompt, options: Optional[GenerationOptions] = None, tools=None, result=None) -> Iterator[str]:
        """Text pieces of one request; the model stays leased until the iterator ends."""
        h = self._of_kind(name, ("text", "chat"))
        o = self._options(h, options)
        start = h.clock()
        i, g, waited = h.acquire()
        try:
            it = g.stream_events(prompt, o, tools, result)
        except QueueFull as e:
            h.release(i)
            h.stats.rejected += 1
            raise InferenceQueueFull(f"model '{name}': {e}") from e

        def pieces():
            ok = False
            try:
                for p in it:
                    yield p
                ok = True
            finally:
                h.release(i)
                h.stats.record(h.clock() - start, waited, ok)
        return pieces()

    def embed(self, name: str, texts: Sequence[str], pooling: str = "mean") -> List[List[float]]:
        h = self._of_kind(name, ("embed", "text", "chat"))

        def run(g):
            out = []
            for t in texts:
                ids = g.tokenizer.encode(t, add_special_tokens=True)
                with g.engine._lock:          # the runner is shared with the generation loop
                    out.append(g.engine.runner.embed_text(ids, pooling).tolist())
            return out
        return h.run(run)

    def count_tokens(self, name: str, text: str) -> int:
        h = self._of_kind(name, ("embed", "text", "chat"))
        return h.run(lambda g: len(g.tokenizer.encode(text, add_special_tokens=True)))

    def invoke(self, name: str, request):
        h = self.model(name)
        call = _PLUGIN_KINDS.get(h.settings.kind)
        if call is None:
            raise TypeError(f"model '{name}' is a {h.settings.kind} model, not a plug-in kind")
        return h.run(lambda m: call(m, request))
