"""Link profiles, calibration, collective-time prediction, throttled transports, capped fake devices and the topology
builder's questions.

    model = LinkCalibration.fit([(bytes, seconds), ...]).link            # least squares: seconds = latency + bytes / bandwidth
    predict_all_reduce(topology, 64 << 20, "hierarchical")               # seconds, from the profiles of the links used
    slow = ThrottledTransport(transport, TokenBucket(rate=1e9, burst=1 << 20))
    devices = carve(total_bytes=16 << 30, parts=4)                       # fake devices with hard memory caps
    TopologyBuilder().build({"nodes": 2, "gpus": 8})                     # answers -> topology document

Reference: src/Idrak.Cluster/Profiles.cs:19 (built-in links), Calibration.cs:46 (least-squares fit),
TopologyInspection.cs:55 (PredictAllReduce), LinkModel.cs:17,67 (TokenBucket, ThrottledTransport),
SimulatedDevices.cs:20 (Carve), TopologyBuilder.cs:113 (questions as data), ClusterCache (calibration files).
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .sim import LinkModel
from .topology import FORMAT, Topology

# latency (s), bandwidth (B/s): NVLink is a measured B200 peer copy through NVSwitch; the rest are typical figures to be replaced by
# a calibration on the machine at hand
BUILT_IN_LINKS: Dict[str, LinkModel] = {
    "sim": LinkModel(0.0, 1e15),
    "nvlink": LinkModel(3e-6, 770e9),
    "pcie-host": LinkModel(8e-6, 50e9),
    "shared-memory": LinkModel(2e-6, 20e9),
    "rdma": LinkModel(4e-6, 45e9),
    "direct-link": LinkModel(30e-6, 10e9),
    "tcp": LinkModel(60e-6, 3e9),
    "udp": LinkModel(80e-6, 1e9),
}
FASTEST_FIRST = ["sim", "nvlink", "pcie-host", "shared-memory", "rdma", "direct-link", "tcp", "udp"]


def fastest(available: Sequence[str]) -> str:
    """The selector's order: the first of ``FASTEST_FIRST`` that is available."""
    for name in FASTEST_FIRST:
        if name in available:
            return name
    raise ValueError(f"none of {list(available)} is a known link type")


# ------------------------------------------------------------------------------------------------ calibration
@dataclass
class LinkCalibration:
    link: LinkModel
    r2: float
    samples: int

    @staticmethod
    def fit(samples: Sequence[Tuple[float, float]]) -> "LinkCalibration":
        """Least squares of seconds against bytes: the intercept is the latency, the slope the inverse bandwidth."""
        pts = [(float(b), float(s)) for b, s in samples]
        if len(pts) < 2 or len({b for b, _ in pts}) < 2:
            raise ValueError("calibration needs measurements at two or more message sizes")
        n = len(pts)
        mx, my = sum(b for b, _ in pts) / n, sum(s for _, s in pts) / n
        sxx = sum((b - mx) ** 2 for b, _ in pts)
        sxy = sum((b - mx) * (s - my) for b, s in pts)
        slope = sxy / sxx
        latency = my - slope * mx
        if slope <= 0:
            raise ValueError("calibration: time does not grow with size; measure larger messages")
        ss_tot = sum((s - my) ** 2 for _, s in pts)
        ss_res = sum((s - (latency + slope * b)) ** 2 for b, s in pts)
        return LinkCalibration(LinkModel(max(latency, 0.0), 1.0 / slope), 1.0 - ss_res / ss_tot if ss_tot > 0 else 1.0, n)


class ClusterCache:
    """Calibrations by link name in one JSON file (next to the tuning decisions)."""

    def __init__(self, path: str):
        self.path = path

    def load(self) -> Dict[str, LinkModel]:
        try:
            with open(self.path, "r", encoding="utf-8") as f:
                doc = json.load(f)
        except (OSError, ValueError):
            return {}
        return {k: LinkModel(**{x: v[x] for x in ("latency", "bandwidth", "jitter", "loss") if x in v})
                for k, v in doc.get("links", {}).items()}

    def store(self, name: str, cal: LinkCalibration) -> None:
        links = {k: asdict(v) for k, v in self.load().items()}
        links[name] = {**asdict(cal.link), "r2": cal.r2, "samples": cal.samples, "measured": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path, "w", encoding="utf-8") as f:
            json.dump({"format": "idrak-cluster-cache/1", "links": links}, f, indent=1)


# ------------------------------------------------------------------------------------------------ prediction
def predict_all_reduce(topology: Topology, nbytes: int, algorithm: str = "ring",
                       links: Optional[Dict[str, LinkModel]] = None) -> float:
    """Seconds for one all-reduce of ``nbytes`` per rank under the link profiles (calibrated ones win over built-in)."""
    table = {**BUILT_IN_LINKS, **(links or {})}
    names = [n.name for n in topology.nodes]
    sizes = [len(n.gpus) for n in topology.nodes]
    w = topology.world
    intra = table[topology.intra_node]
    cross = [table[topology.link_type(a, b)] for i, a in enumerate(names) for b in names[i + 1:]]
    slow_cross = min(cross, key=lambda l: l.bandwidth) if cross else None
    slowest = min([intra] + cross, key=lambda l: l.bandwidth) if (cross and max(sizes) > 1) else (slow_cross or intra)
    if w == 1:
        return 0.0
    if algorithm == "naive":
        return 2 * (w - 1) * slowest.transfer_time(nbytes)            # the first rank receives, then sends, one by one
    if algorithm == "ring":
        return 2 * (w - 1) * slowest.transfer_time(nbytes / w)
    if algorithm == "hierarchical":
        c, m = min(sizes), len(names)
        t = 0.0
        if max(sizes) > c:
            t += 2 * intra.transfer_time(nbytes)                        # extra ranks hand over and get the result back
        if c > 1:
            t += 2 * (c - 1) * intra.transfer_time(nbytes / c)
        if m > 1:
            t += 2 * (m - 1) * slow_cross.transfer_time(nbytes / c / m)
        return t
    raise KeyError(f"Collective algorithm '{algorithm}' is not registered. Known: hierarchical, naive, ring")


# ------------------------------------------------------------------------------------------------ throttling
class TokenBucket:
    """``rate`` bytes per second with ``burst`` bytes of credit; ``take`` returns how long the caller has to wait."""

    def __init__(self, rate: float, burst: float, clock: Callable[[], float] = time.monotonic):
        if rate <= 0 or burst <= 0:
            raise ValueError("rate and burst must be positive")
        self.rate, self.burst, self.clock = float(rate), float(burst), clock
        self.credit, self.at = float(burst), clock()

    def take(self, nbytes: float) -> float:
        now = self.clock()
        self.credit = min(self.burst, self.credit + (now - self.at) * self.rate)
        self.at = now
        self.credit -= nbytes                                          # may go negative: the debt is the wait
        return max(0.0, -self.credit / self.rate)


class ThrottledTransport:
    """A transport of ``parallel.host_collectives`` slowed to a token bucket and a fixed latency per message."""

    def __init__(self, inner, bucket: TokenBucket, latency: float = 0.0, sleep: Callable[[float], None] = time.sleep):
        self.inner, self.bucket, self.latency, self.sleep = inner, bucket, latency, sleep
        self.rank, self.world = inner.rank, inner.world
        self.waited = 0.0

    def exchange(self, dst, out, src, count, dtype):
        if dst is not None:
            wait = self.latency + self.bucket.take(out.numel() * out.element_size())
            if wait > 0:
                self.waited += wait
                self.sleep(wait)
        return self.inner.exchange(dst, out, src, count, dtype)


# ------------------------------------------------------------------------------------------------ fake devices
class DeviceMemoryExceeded(MemoryError):
    pass


class SimulatedDevice:
    """A share of one physical device with a hard cap; allocations beyond it fail like the real thing would."""

    def __init__(self, name: str, capacity: int):
        self.name, self.capacity, self.used, self.peak = name, int(capacity), 0, 0

    def allocate(self, nbytes: int) -> int:
        if self.used + nbytes > self.capacity:
            raise DeviceMemoryExceeded(f"{self.name}: {nbytes} bytes asked, {self.capacity - self.used} of {self.capacity} free")
        self.used += int(nbytes)
        self.peak = max(self.peak, self.used)
        return self.used

    def release(self, nbytes: int) -> None:
        self.used = max(0, self.used - int(nbytes))


def carve(total_bytes: int, parts: int, reserve: float = 0.05) -> List[SimulatedDevice]:
    """Split one device's memory into ``parts`` equal fake devices, keeping ``reserve`` of it for the real runtime."""
    if parts <= 0:
        raise ValueError("parts must be positive")
    each = int(total_bytes * (1.0 - reserve)) // parts
    return [SimulatedDevice(f"sim:{i}", each) for i in range(parts)]


# ------------------------------------------------------------------------------------------------ builder
class TopologyBuilder:
    """The questions a front end asks, as data, and the document their answers give."""

    QUESTIONS = [
        {"key": "nodes", "prompt": "How many machines?", "kind": "int", "default": 1, "min": 1},
        {"key": "gpus", "prompt": "GPUs per machine?", "kind": "int", "default": 8, "min": 1},
        {"key": "memory", "prompt": "Memory per GPU?", "kind": "text", "default": "180GiB"},
        {"key": "addresses", "prompt": "Addresses of the machines (comma separated)?", "kind": "text", "default": "",
         "when": lambda a: int(a.get("nodes", 1)) > 1},
        {"key": "inter_node", "prompt": "Link between machines?", "kind": "choice", "default": "tcp",
         "choices": ["rdma", "direct-link", "tcp"], "when": lambda a: int(a.get("nodes", 1)) > 1},
    ]

    def questions(self, answers: Optional[dict] = None) -> List[dict]:
        answers = answers or {}
        return [{k: v for k, v in q.items() if k != "when"} for q in self.QUESTIONS if q.get("when", lambda a: True)(answers)]

    def build(self, answers: dict) -> dict:
        a = {q["key"]: answers.get(q["key"], q["default"]) for q in self.QUESTIONS}
        nodes, gpus = int(a["nodes"]), int(a["gpus"])
        if nodes < 1 or gpus < 1:
            raise ValueError("nodes and gpus must be at least 1")
        addresses = [x.strip() for x in str(a["addresses"]).split(",") if x.strip()]
        if addresses and len(addresses) != nodes:
            raise ValueError(f"{len(addresses)} addresses for {nodes} machines")
        if a["inter_node"] not in BUILT_IN_LINKS:
            raise ValueError(f"unknown link type '{a['inter_node']}'")
        return {"format": FORMAT,
                "nodes": [{"name": f"node{i}", "address": addresses[i] if addresses else ("127.0.0.1" if nodes == 1 else f"10.0.0.{i + 1}"),
                           "gpus": [{"device": g, "memory": a["memory"]} for g in range(gpus)]} for i in range(nodes)],
                "links": {"intra-node": "nvlink", "inter-node": a["inter_node"]}}
