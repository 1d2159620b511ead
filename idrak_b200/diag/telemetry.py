"""Telemetry bus: levels as bit flags, typed events, hooks.

``Telemetry.is_enabled(level)`` is one attribute read and an AND, so publish sites cost nothing when
nobody listens. Hooks receive every event whose level they subscribed to: ``ConsoleLogger``,
``MetricsRecorder`` (per-step series), ``JsonLinesLogger`` (``log.jsonl``), ``ChannelTelemetry`` (a queue).

Reference: Telemetry (src/Idrak.Abstraction/Diagnostics/Telemetry.cs:11-91,290,327), Events.cs:18-705,
Hooks.cs:20,257,444,583,743.
"""
from __future__ import annotations

import dataclasses
import enum
import json
import queue
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional


class Level(enum.IntFlag):
    NONE = 0
    TRAINING = 1 << 0
    BATCHES = 1 << 1
    GRADIENTS = 1 << 2
    LAYERS = 1 << 3
    OPERATIONS = 1 << 4
    INFERENCE = 1 << 5
    TOOLS = 1 << 6
    ENGINE = 1 << 7
    DEVICES = 1 << 8
    OVERRIDES = 1 << 9
    SUGGESTIONS = 1 << 10
    NETWORK = 1 << 11
    STAGES = 1 << 12
    MCP = 1 << 13
    ALL = (1 << 14) - 1

    @classmethod
    def parse(cls, text: str) -> "Level":
        out = cls.NONE
        for part in text.replace("|", ",").split(","):
            part = part.strip()
            if not part:
                continue
            try:
                out |= cls[part.upper()]
            except KeyError:
                raise ValueError(f"unknown telemetry level '{part}' (one of {[m.name.lower() for m in cls]})")
        return out


# --------------------------------------------------------------------------- events
@dataclass
class Event:
    kind: str = ""
    time: float = field(default_factory=time.time)
    data: Dict[str, Any] = field(default_factory=dict)

    def to_json(self) -> dict:
        d = {k: v for k, v in dataclasses.asdict(self).items() if k not in ("data",)}
        d.update(self.data)
        d["kind"] = self.kind or type(self).__name__
        return d


@dataclass
class BatchCompleted(Event):
    epoch: int = 0
    step: int = 0
    loss: float = 0.0
    size: int = 0
    tokens: int = 0
    seconds: float = 0.0


@dataclass
class EpochCompleted(Event):
    epoch: int = 0
    loss: float = 0.0
    validation_loss: Optional[float] = None
    metrics: Dict[str, float] = field(default_factory=dict)
    validation_metrics: Dict[str, float] = field(default_factory=dict)
    learning_rate: float = 0.0
    seconds: float = 0.0
    samples: int = 0


@dataclass
class OperationCompleted(Event):
    name: str = ""
    microseconds: float = 0.0
    flops: float = 0.0
    bytes: float = 0.0


@dataclass
class CollectiveCompleted(Event):
    op: str = ""
    algorithm: str = ""
    bytes: int = 0
    ranks: int = 0
    microseconds: float = 0.0


@dataclass
class GradientsSynced(Event):
    step: int = 0
    buckets: int = 0
    bytes: int = 0
    exposed_microseconds: float = 0.0


@dataclass
class EngineEvent(Event):
    model: str = ""
    what: str = ""           # loaded | unloaded | queued | rejected | leased | completed | failed
    queue: int = 0
    milliseconds: float = 0.0


@dataclass
class InferenceStage(Event):
    stage: str = ""          # prefill | decode | sample
    tokens: int = 0
    milliseconds: float = 0.0


@dataclass
class DeviceFailed(Event):
    device: str = ""
    operation: str = ""
    message: str = ""
    hint: str = ""


@dataclass
class RankStateChanged(Event):
    rank: int = 0
    state: str = ""


@dataclass
class FaultInjected(Event):
    fault: str = ""
    rank: int = 0
    step: int = 0
    seed: int = 0


@dataclass
class SettingSuggestion(Event):
    setting: str = ""
    value: str = ""
    reason: str = ""


@dataclass
class TuningCompleted(Event):
    shape_class: str = ""
    choice: str = ""
    candidates: int = 0
    microseconds: float = 0.0


# --------------------------------------------------------------------------- hooks
class TelemetryHook:
    levels: Level = Level.ALL

    def handle(self, level: Level, event: Event) -> None:
        raise NotImplementedError


class ConsoleLogger(TelemetryHook):
    def __init__(self, levels: Level = Level.TRAINING, stream=None):
        self.levels, self.stream = levels, stream or sys.stderr

    def handle(self, level, event):
        d = event.to_json()
        kind = d.pop("kind")
        d.pop("time", None)
        body = " ".join(f"{k}={v:.5g}" if isinstance(v, float) else f"{k}={v}" for k, v in d.items()
                        if v not in (None, {}, []))
        print(f"[{level.name.lower()}] {kind} {body}", file=self.stream)


class JsonLinesLogger(TelemetryHook):
    def __init__(self, path, levels: Level = Level.ALL):
        self.levels = levels
        self._f = open(path, "a", buffering=1)
        self._lock = threading.Lock()

    def handle(self, level, event):
        d = event.to_json()
        d["level"] = level.name.lower()
        with self._lock:
            self._f.write(json.dumps(d, default=str) + "\n")

    def close(self):
        self._f.close()


class MetricsRecorder(TelemetryHook):
    """Per-step series: loss, learning rate, gradient norm, tokens/s, collectives ..."""

    def __init__(self, levels: Level = Level.TRAINING | Level.BATCHES | Level.NETWORK | Level.GRADIENTS):
        self.levels = levels
        self.series: Dict[str, List[float]] = {}
        self.events: List[Event] = []

    def handle(self, level, event):
        self.events.append(event)
        for k, v in event.to_json().items():
            if isinstance(v, (int, float)) and not isinstance(v, bool) and k != "time":
                self.series.setdefault(f"{type(event).__name__}.{k}", []).append(float(v))


class ChannelTelemetry(TelemetryHook):
    def __init__(self, levels: Level = Level.ALL, capacity: int = 4096):
        self.levels = levels
        self.queue: "queue.Queue[tuple[Level, Event]]" = queue.Queue(capacity)

    def handle(self, level, event):
        try:
            self.queue.put_nowait((level, event))
        except queue.Full:
            pass


# --------------------------------------------------------------------------- bus
class _Bus:
    def __init__(self):
        self.enabled: int = 0
        self._hooks: List[TelemetryHook] = []
        self._lock = threading.Lock()

    def is_enabled(self, level: Level) -> bool:
        return (self.enabled & int(level)) != 0

    def add(self, hook: TelemetryHook) -> TelemetryHook:
        with self._lock:
            self._hooks.append(hook)
            self.enabled |= int(hook.levels)
        return hook

    def remove(self, hook: TelemetryHook) -> None:
        with self._lock:
            if hook in self._hooks:
                self._hooks.remove(hook)
            self.enabled = 0
            for h in self._hooks:
                self.enabled |= int(h.levels)

    def publish_event(self, level: Level, event: Event) -> None:
        if not (self.enabled & int(level)):
            return
        for h in list(self._hooks):
            if int(h.levels) & int(level):
                h.handle(level, event)

    def publish(self, level: Level, kind: str, **data) -> None:
        if not (self.enabled & int(level)):
            return
        self.publish_event(level, Event(kind=kind, data=data))

    def clear(self):
        with self._lock:
            self._hooks.clear()
            self.enabled = 0


Telemetry = _Bus()
