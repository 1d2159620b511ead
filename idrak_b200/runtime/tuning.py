"""Per-device measured tuning. The first time a shape class needs a choice (how many ways to split K, which tile
shape), every candidate is timed on the real inputs; the winner must beat the default by a margin to be taken, and the
decision is stored per GPU + driver + library build so later processes start with it.

Timing: candidates are run interleaved (A B C A B C ...) after a warm-up, each run timed with CUDA events; a
candidate's figure is the median of its per-round ratios to the default in the same round, which cancels clock drift
between rounds. Decode-sized work can be timed with a cold L2 (a buffer larger than L2 is rewritten before each
run). A candidate replaces the default only when its median ratio is below ``1 - min_win`` (3 % by default).

    choice = tuner().choose("gemm.splits", (64, 6144, 4096), {"1": f1, "4": f4, "6": f6}, default="6", cold_l2=True)

Settings: ``IDRAK_AUTOTUNE`` (off: always the default; the cache is still read), ``IDRAK_TUNING_CACHE`` (file path).

Reference: the reference's tuning cache (src/Idrak.Gpu/Cuda/TuningCache.cs, CudaBackend.Tuning.cs:1-40: median of paired
ratios, at least 3 % to win, cold-L2 timing for decode-sized products, one file per GPU + driver + build; TuneSizes.cs
size classes).
"""
from __future__ import annotations

import json
import os
import statistics
import threading
from typing import Callable, Dict, Iterable, Optional, Sequence, Tuple

from .. import config

_lock = threading.Lock()
_tuner: Optional["Tuner"] = None


def size_class(n: int) -> int:
    """Sizes that share a tuning decision: the next power of two at or above ``n`` (1, 2, 4, ... ), so 48 and 64 rows
    choose together while 65 rows do not."""
    c = 1
    while c < n:
        c <<= 1
    return c


def device_key() -> str:
    """GPU name, driver and library build: a decision measured on one does not carry to another."""
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(torch.cuda.current_device())
            from .. import _native
            build = _native.lib().idrak_build_info().decode() if _native.available() else "no-native"
            return f"{p.name}|sm{p.major}{p.minor}|{p.multi_processor_count}sm|cuda{torch.version.cuda}|{build}"
    except Exception:
        pass
    return "cpu"


def _time_cuda(fn: Callable[[], None], flush) -> float:
    import torch
    if flush is not None:
        flush.fill_(1)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


class Tuner:
    def __init__(self, path: Optional[str] = None, enabled: Optional[bool] = None, key: Optional[str] = None,
                 timer: Optional[Callable[[Callable[[], None], object], float]] = None):
        self.path = path if path is not None else (config.get("IDRAK_TUNING_CACHE") or
                                                   os.path.join(config.get("IDRAK_HOME"), "tuning.json"))
        self.enabled = config.get("IDRAK_AUTOTUNE") if enabled is None else enabled
        self.key = key or device_key()
        self.timer = timer or _time_cuda
        self.table: Dict[str, Dict[str, dict]] = {}
        self.measured = 0
        self._flush = None
        self._load()

    # ------------------------------------------------------------------ the file
    def _load(self) -> None:
        try:
            with open(self.path, "r", encoding="utf-8") as f:
                doc = json.load(f)
            if doc.get("format") == "idrak-tuning/1":
                self.table = doc.get("devices", {})
        except (OSError, ValueError):
            self.table = {}

    def save(self) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(self.path)) or ".", exist_ok=True)
        tmp = f"{self.path}.{os.getpid()}.tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump({"format": "idrak-tuning/1", "devices": self.table}, f, indent=1, sort_keys=True)
        os.replace(tmp, self.path)

    def entries(self) -> Dict[str, dict]:
        return dict(self.table.get(self.key, {}))

    def forget(self, prefix: str = "") -> int:
        mine = self.table.get(self.key, {})
        drop = [k for k in mine if k.startswith(prefix)]
        for k in drop:
            del mine[k]
        if drop:
            self.save()
        return len(drop)

    # ------------------------------------------------------------------ decisions
    @staticmethod
    def entry_name(kind: str, shape: Sequence[int]) -> str:
        return f"{kind}:" + "x".join(str(int(v)) for v in shape)

    def lookup(self, kind: str, shape: Sequence[int]) -> Optional[str]:
        e = self.table.get(self.key, {}).get(self.entry_name(kind, shape))
        return None if e is None else e["choice"]

    def choose(self, kind: str, shape: Sequence[int], candidates: Dict[str, Callable[[], None]], default: str,
               min_win: float = 0.03, rounds: int = 7, warmup: int = 2, cold_l2: bool = False) -> str:
        """The stored decision for (kind, shape); else, when tuning is on, measure the candidates, store and return the
        winner; else the default."""
        known = self.lookup(kind, shape)
        if known is not None and known in candidates:
            return known
        if not self.enabled or len(candidates) < 2:
            return default
        if default not in candidates:
            raise KeyError(f"the default '{default}' is not among the candidates")
        with _lock:
            flush = self._flush_buffer() if cold_l2 else None
            names = [default] + [n for n in candidates if n != default]
            for _ in range(warmup):
                for n in names:
                    candidates[n]()
            ratios: Dict[str, list] = {n: [] for n in names[1:]}
            base_ms = []
            for _ in range(rounds):
                times = {n: self.timer(candidates[n], flush) for n in names}
                base_ms.append(times[default])
                for n in names[1:]:
                    ratios[n].append(times[n] / max(times[default], 1e-9))
            medians = {n: statistics.median(r) for n, r in ratios.items()}
            best = min(medians, key=medians.get)
            choice = best if medians[best] < 1.0 - min_win else default
            self.measured += 1
            self.table.setdefault(self.key, {})[self.entry_name(kind, shape)] = {
                "choice": choice, "default": default, "default_ms": round(statistics.median(base_ms), 5),
                "ratios": {n: round(v, 4) for n, v in medians.items()}, "cold_l2": bool(cold_l2)}
            self.save()
            return choice

    def _flush_buffer(self):
        if self._flush is None:
            import torch
            self._flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        return self._flush


def tuner() -> Tuner:
    global _tuner
    if _tuner is None:
        _tuner = Tuner()
    return _tuner


def reset_tuner() -> None:
    global _tuner
    _tuner = None
