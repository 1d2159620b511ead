"""Profiling: a kernel-level GPU profiler (device time per kernel name, launches, share of the total, TFLOP/s where the
FLOPs are known) and a ``Profiler`` that runs a piece of work cold and warm and reports wall time, device time, memory
and the kernel table, with writers for a text table, Markdown, CSV and JSON.

    report = Profiler.run("train step", lambda: step(ids, targets), warm=5)
    print(report.table())

    with GpuProfiler() as gp:
        step(ids, targets)
    for row in gp.rows()[:10]: ...

On CUDA the kernel times come from the profiler of the tensor library (CUPTI activity records); on the CPU the
operator times of the same profiler stand in. Numbers taken under this profiler are for attribution (shares), not
headline throughput - the benchmarks time with CUDA events and no profiler attached.

Reference: Profiler.Run / ProfileReport / ProfileProbes (src/Idrak.Abstraction/Diagnostics/Profiling.cs:427,696) and
GpuProfiler (src/Idrak/Diagnostics/GpuProfiler.cs:19: every launch bracketed by events, keyed by kernel name, TFLOPS tables).
"""
from __future__ import annotations

import csv
import io
import json
import re
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional

import torch


@dataclass
class KernelRow:
    name: str
    launches: int
    total_us: float
    mean_us: float
    share: float
    tflops: Optional[float] = None


def _short(name: str) -> str:
    name = re.sub(r"^void\s+", "", name)
    name = re.sub(r"\(.*$", "", name)
    return name.replace("idrak::", "")


class GpuProfiler:
    """Collect device time per kernel between ``start`` and ``stop`` (or inside a ``with`` block)."""

    def __init__(self, flops: Optional[Dict[str, float]] = None):
        self.flops = flops or {}            # kernel-name substring -> FLOPs per launch
        self._prof = None
        self._rows: List[KernelRow] = []

    def start(self) -> "GpuProfiler":
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts)
        self._prof.__enter__()
        return self

    def stop(self) -> List[KernelRow]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        cuda = torch.cuda.is_available()
        agg: Dict[str, List[float]] = {}
        for ev in self._prof.events():
            if cuda:
                if ev.device_type != torch.autograd.DeviceType.CUDA:
                    continue
                dur = float(getattr(ev, "device_time", 0.0) or getattr(ev, "cuda_time", 0.0) or 0.0)
            else:
                dur = float(getattr(ev, "self_cpu_time_total", 0.0))
                if dur <= 0:
                    continue
            a = agg.setdefault(_short(ev.name), [0, 0.0])
            a[0] += 1
            a[1] += dur
        total = sum(v[1] for v in agg.values()) or 1.0
        rows = []
        for name, (n, us) in agg.items():
            fl = next((f for key, f in self.flops.items() if key in name), None)
            rows.append(KernelRow(name, n, us, us / n, us / total, (fl * n / (us * 1e-6) / 1e12) if fl and us > 0 else None))
        self._rows = sorted(rows, key=lambda r: -r.total_us)
        return self._rows

    def rows(self) -> List[KernelRow]:
        return list(self._rows)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False


@dataclass
class ProfileReport:
    name: str
    device: str
    cold_ms: List[float] = field(default_factory=list)
    warm_ms: List[float] = field(default_factory=list)
    warm_device_ms: List[float] = field(default_factory=list)
    peak_memory_bytes: int = 0
    kernels: List[KernelRow] = field(default_factory=list)

    @property
    def warm_median_ms(self) -> float:
        s = sorted(self.warm_ms)
        return s[len(s) // 2] if s else float("nan")

    # ------------------------------------------------------------------ writers
    def to_json(self) -> str:
        d = asdict(self)
        d["warm_median_ms"] = self.warm_median_ms
        return json.dumps(d)

    def to_csv(self) -> str:
        buf = io.StringIO()
        w = csv.writer(buf)
        w.writerow(["kernel", "launches", "total_us", "mean_us", "share", "tflops"])
        for r in self.kernels:
            w.writerow([r.name, r.launches, f"{r.total_us:.1f}", f"{r.mean_us:.2f}", f"{r.share:.4f}",
                        "" if r.tflops is None else f"{r.tflops:.1f}"])
        return buf.getvalue()

    def _summary(self) -> List[str]:
        lines = [f"{self.name} on {self.device}"]
        if self.cold_ms:
            lines.append(f"cold  {', '.join(f'{v:.2f}' for v in self.cold_ms)} ms")
        if self.warm_ms:
            lines.append(f"warm  median {self.warm_median_ms:.3f} ms over {len(self.warm_ms)} runs"
                         + (f"; device {sorted(self.warm_device_ms)[len(self.warm_device_ms) // 2]:.3f} ms" if self.warm_device_ms else ""))
        if self.peak_memory_bytes:
            lines.append(f"peak memory {self.peak_memory_bytes / 2 ** 20:.1f} MiB")
        return lines

    def table(self, top: int = 20) -> str:
        lines = self._summary()
        if self.kernels:
            width = min(max(len(r.name) for r in self.kernels[:top]), 60)
            lines.append(f"{'kernel'.ljust(width)}  launches   total us   mean us  share  TFLOP/s")
            for r in self.kernels[:top]:
                lines.append(f"{r.name[:width].ljust(width)}  {r.launches:8d}  {r.total_us:9.1f}  {r.mean_us:8.2f}  {100 * r.share:4.1f}%"
                             + ("" if r.tflops is None else f"  {r.tflops:7.1f}"))
        return "\n".join(lines)

    def to_markdown(self, top: int = 20) -> str:
        lines = [f"### {self.name}", ""] + [f"* {s}" for s in self._summary()[1:]] + [""]
        if self.kernels:
            lines += ["| kernel | launches | total us | mean us | share | TFLOP/s |", "|---|---|---|---|---|---|"]
            for r in self.kernels[:top]:
                lines.append(f"| `{r.name}` | {r.launches} | {r.total_us:.1f} | {r.mean_us:.2f} | {100 * r.share:.1f} % | "
                             f"{'' if r.tflops is None else f'{r.tflops:.1f}'} |")
        return "\n".join(lines)


class Profiler:
    @staticmethod
    def run(name: str, work: Callable[[], object], cold: int = 1, warm: int = 5, kernels: bool = True,
            flops: Optional[Dict[str, float]] = None, device: Optional[str] = None) -> ProfileReport:
        """Run ``work`` ``cold`` times first (lazy initialisation, cold caches: kept apart), then ``warm`` times timed by
        wall clock and CUDA events, then once more under the kernel profiler."""
        cuda = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
        rep = ProfileReport(name, torch.cuda.get_device_name() if cuda else "cpu")

        def sync():
            if cuda:
                torch.cuda.synchronize()

        for _ in range(cold):
            sync()
            t0 = time.perf_counter()
            work()
            sync()
            rep.cold_ms.append((time.perf_counter() - t0) * 1e3)
        if cuda:
            torch.cuda.reset_peak_memory_stats()
        for _ in range(warm):
            sync()
            if cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            t0 = time.perf_counter()
            work()
            if cuda:
                b.record()
            sync()
            rep.warm_ms.append((time.perf_counter() - t0) * 1e3)
            if cuda:
                rep.warm_device_ms.append(a.elapsed_time(b))
        if cuda:
            rep.peak_memory_bytes = int(torch.cuda.max_memory_allocated())
        if kernels:
            with GpuProfiler(flops) as gp:
                work()
            rep.kernels = gp.rows()
        return rep
