"""A cluster in one process: rank threads, a transport with a link model on a virtual clock, seeded failures and
a replayable event log. For testing what happens around the kernels - timeouts that name the rank, stop agreement,
late joiners, slow or dropped workers - without touching a GPU.

    def rank_main(ctx):                      # ctx.rank, ctx.world, ctx.send / recv / all_reduce / barrier
        total = ctx.all_reduce([float(ctx.rank)])
    result = InProcessCluster(world=4, link=LinkModel(latency=5e-6, bandwidth=50e9),
                              failures=FaultInjector(seed=3, model="slow-worker")).run(rank_main, steps=10)

Time is virtual: a message of ``n`` bytes arrives ``latency + n / bandwidth (+ jitter)`` after it was sent on the
sender's clock, a receiver's clock jumps to the arrival time, so runs repeat exactly and a 120-second timeout costs
no wall time. Every fault is drawn from ``(seed, step, rank)`` and logged with that key; ``ClusterReplay`` feeds a
log back so a failing run can be repeated.

Reference: InProcessCluster / SimTransport / VirtualClock / FaultInjector / EventLog / ClusterReplay
(src/Idrak.Network/Cluster/*.cs; failure models Failures.cs:86-124).
"""
from __future__ import annotations

import json
import queue
import struct
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

FAILURE_MODELS = ("none", "slow-worker", "dropped-worker", "link-loss", "partition", "late-join", "mixed")


class RankTimeout(TimeoutError):
    """A wait on another rank ran out; the message names the rank."""

    def __init__(self, waiting: int, on: int, seconds: float, what: str):
        super().__init__(f"rank {waiting}: no {what} from rank {on} within {seconds:g} s")
        self.waiting, self.on = waiting, on


class RankDropped(RuntimeError):
    """Raised inside a rank the failure model removed from the run."""


@dataclass
class LinkModel:
    latency: float = 5e-6            # seconds
    bandwidth: float = 50e9          # bytes per second
    jitter: float = 0.0              # up to this share of the transfer time is added, seeded
    loss: float = 0.0                # probability that a message is lost (the receiver times out)

    def transfer_time(self, nbytes: int, u: float = 0.0) -> float:
        t = self.latency + nbytes / self.bandwidth
        return t * (1.0 + self.jitter * u)


@dataclass
class Fault:
    step: int
    rank: int
    kind: str                        # slow | drop | loss | partition | late
    amount: float = 0.0              # slow: seconds added; late: steps sat out
    peer: int = -1

    def key(self) -> str:
        return f"{self.kind}@step{self.step}/rank{self.rank}" + (f"->{self.peer}" if self.peer >= 0 else "")


class FaultInjector:
    """Draws the faults of a step from ``(seed, step)``; the same seed gives the same run."""

    def __init__(self, seed: int = 0, model: str = "none", rate: float = 0.2, slow_seconds: float = 0.5,
                 scripted: Optional[Sequence[Fault]] = None):
        if model not in FAILURE_MODELS and model != "scripted":
            raise KeyError(f"Failure model '{model}' is not registered. Known: {', '.join(FAILURE_MODELS)}")
        self.seed, self.model, self.rate, self.slow_seconds = seed, model, rate, slow_seconds
        self.scripted = list(scripted or [])

    def faults(self, step: int, world: int) -> List[Fault]:
        if self.model == "scripted":
            return [f for f in self.scripted if f.step == step]
        if self.model == "none":
            return []
        rng = np.random.default_rng([self.seed, step])
        kinds = {"slow-worker": ["slow"], "dropped-worker": ["drop"], "link-loss": ["loss"], "partition": ["partition"],
                 "late-join": ["late"], "mixed": ["slow", "loss", "late"]}[self.model]
        out = []
        if rng.random() < self.rate:
            kind = kinds[int(rng.integers(0, len(kinds)))]
            rank = int(rng.integers(1 if kind in ("drop", "late") else 0, world))
            peer = int((rank + 1 + rng.integers(0, world - 1)) % world) if kind in ("loss", "partition") else -1
            amount = self.slow_seconds * (1 + rng.random()) if kind == "slow" else (1 + int(rng.integers(0, 3))
                                                                                      if kind == "late" else 0.0)
            out.append(Fault(step, rank, kind, float(amount), peer))
        return out


class EventLog:
    """Append-only record of a run: one record per event, binary (length-prefixed JSON) so it can be streamed."""

    MAGIC = b"IKEV1\n"

    def __init__(self):
        self.events: List[dict] = []
        self._lock = threading.Lock()

    def add(self, kind: str, **fields) -> None:
        with self._lock:
            self.events.append({"kind": kind, **fields})

    def of(self, kind: str) -> List[dict]:
        return [e for e in self.events if e["kind"] == kind]

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.MAGIC)
            for e in self.events:
                raw = json.dumps(e, sort_keys=True).encode()
                f.write(struct.pack("<I", len(raw)) + raw)

    @classmethod
    def load(cls, path: str) -> "EventLog":
        log = cls()
        with open(path, "rb") as f:
            if f.read(len(cls.MAGIC)) != cls.MAGIC:
                raise ValueError(f"{path}: not an event log")
            while True:
                head = f.read(4)
                if not head:
                    break
                (n,) = struct.unpack("<I", head)
                log.events.append(json.loads(f.read(n)))
        return log


class SimTransport:
    """Bounded in-process queues between rank threads; delivery times follow the link model on virtual clocks."""

    def __init__(self, world: int, link: LinkModel, seed: int = 0, timeout: float = 120.0, wall_timeout: float = 20.0,
                 capacity: int = 64):
        self.world, self.link, self.timeout, self.wall_timeout = world, link, timeout, wall_timeout
        self.queues = {(s, d): queue.Queue(maxsize=capacity) for s in range(world) for d in range(world) if s != d}
        self.clock = [0.0] * world                   # virtual seconds, one clock per rank
        self.cut: set = set()                        # (a, b) pairs that cannot talk (partition / link loss)
        self.gone: set = set()                       # ranks that left without saying so
        self.seed = int(seed)
        self._sent: Dict[Tuple[int, int], int] = {}
        self._lock = threading.Lock()
        self.bytes_sent = 0
        self.messages = 0

    def send(self, src: int, dst: int, payload: Any, nbytes: int) -> None:
        with self._lock:
            n = self._sent.get((src, dst), 0)
            self._sent[(src, dst)] = n + 1
            self.bytes_sent += nbytes
            self.messages += 1
        # jitter and loss are a function of (seed, pair, message number), not of which thread got here first
        draw = np.random.default_rng([self.seed, src, dst, n]).random(2)
        u, lost = float(draw[0]), bool(draw[1] < self.link.loss)
        arrival = self.clock[src] + self.link.transfer_time(nbytes, u)
        if lost or (src, dst) in self.cut or (dst, src) in self.cut:
            return                                   # the receiver will run into its timeout
        self.queues[(src, dst)].put((arrival, payload))

    def recv(self, dst: int, src: int, what: str = "message") -> Any:
        waited = 0.0
        while True:
            try:
                arrival, payload = self.queues[(src, dst)].get(timeout=0.02)
                self.clock[dst] = max(self.clock[dst], arrival)
                return payload
            except queue.Empty:
                waited += 0.02
                unreachable = src in self.gone or (src, dst) in self.cut or (dst, src) in self.cut
                if unreachable or waited >= self.wall_timeout:
                    # on the virtual clock the whole timeout has passed
                    self.clock[dst] += self.timeout
                    raise RankTimeout(dst, src, self.timeout, what)


class RankContext:
    """What a rank's code sees: point-to-point messages and the collectives built on them (rank-ordered sums)."""

    def __init__(self, rank: int, world: int, transport: SimTransport, log: EventLog):
        self.rank, self.world, self.transport, self.log = rank, world, transport, log
        self.step = 0
        self.members = list(range(world))            # ranks taking part in the current step

    # ---- time
    @property
    def now(self) -> float:
        return self.transport.clock[self.rank]

    def compute(self, seconds: float) -> None:
        self.transport.clock[self.rank] += seconds

    # ---- messages
    def send(self, dst: int, payload: Any, nbytes: Optional[int] = None) -> None:
        n = nbytes if nbytes is not None else (payload.nbytes if hasattr(payload, "nbytes") else 64)
        self.transport.send(self.rank, dst, payload, int(n))

    def recv(self, src: int, what: str = "message") -> Any:
        return self.transport.recv(self.rank, src, what)

    # ---- collectives over the current members
    def all_reduce(self, values, op: str = "sum") -> np.ndarray:
        """Gather at the lowest member, reduce in rank order, broadcast: identical bits on every rank."""
        v = np.asarray(values, dtype=np.float64)
        root = self.members[0]
        if self.rank == root:
            parts = {root: v}
            for r in self.members[1:]:
                parts[r] = self.recv(r, "all-reduce part")
            total = parts[self.members[0]].copy()
            for r in self.members[1:]:
                total = np.maximum(total, parts[r]) if op == "max" else total + parts[r]
            for r in self.members[1:]:
                self.send(r, total, total.nbytes)
            return total
        self.send(root, v, v.nbytes)
        return self.recv(root, "all-reduce result")

    def barrier(self) -> None:
        self.all_reduce([0.0])

    def broadcast(self, value, root: int = 0):
        if self.rank == root:
            for r in self.members:
                if r != root:
                    self.send(r, value)
            return value
        return self.recv(root, "broadcast")


@dataclass
class ClusterResult:
    returns: Dict[int, Any]
    errors: Dict[int, BaseException]
    log: EventLog
    virtual_seconds: float
    bytes_sent: int


class InProcessCluster:
    """Runs ``fn(ctx, step)`` for ``steps`` steps on every rank thread, applying the failure model between steps."""

    def __init__(self, world: int, link: Optional[LinkModel] = None, failures: Optional[FaultInjector] = None,
                 seed: int = 0, timeout: float = 120.0, wall_timeout: float = 20.0):
        self.world = world
        self.link = link or LinkModel()
        self.failures = failures or FaultInjector()
        self.log = EventLog()
        self.transport = SimTransport(world, self.link, seed, timeout, wall_timeout)

    def run(self, fn: Callable[[RankContext, int], Any], steps: int = 1) -> ClusterResult:
        returns: Dict[int, Any] = {}
        errors: Dict[int, BaseException] = {}
        plan = {s: self.failures.faults(s, self.world) for s in range(steps)}
        for s, faults in plan.items():
            for f in faults:
                self.log.add("fault", step=f.step, rank=f.rank, fault=f.kind, amount=f.amount, peer=f.peer, key=f.key())
        # who sits out which steps (late joiners), who leaves for good
        sits_out = {r: set() for r in range(self.world)}
        leaves_at: Dict[int, int] = {}
        for s, faults in plan.items():
            for f in faults:
                if f.kind == "late":
                    sits_out[f.rank].update(range(s, min(steps, s + int(f.amount))))
                if f.kind == "drop":
                    leaves_at.setdefault(f.rank, s)

        def members_of(step: int) -> List[int]:
            return [r for r in range(self.world) if step not in sits_out[r]]

        def main(rank: int):
            ctx = RankContext(rank, self.world, self.transport, self.log)
            try:
                out = None
                for step in range(steps):
                    ctx.step = step
                    if rank in leaves_at and step >= leaves_at[rank]:
                        self.transport.gone.add(rank)
                        self.log.add("left", step=step, rank=rank)
                        raise RankDropped(f"rank {rank} dropped at step {step}")
                    for f in plan[step]:
                        if f.kind == "slow" and f.rank == rank:
                            ctx.compute(f.amount)
                        if f.kind in ("loss", "partition") and f.rank == rank:
                            self.transport.cut.add((f.rank, f.peer))
                    # dropped ranks stay in the member list: the others find out by their timeout
                    ctx.members = members_of(step)
                    if rank not in ctx.members:
                        self.log.add("sat-out", step=step, rank=rank)
                        continue
                    out = fn(ctx, step)
                returns[rank] = out
            except BaseException as e:       # recorded per rank; the launcher decides what a failure means
                errors[rank] = e
                self.transport.gone.add(rank)      # a rank that ended ends every wait on it at once
                self.log.add("error", rank=rank, step=ctx.step, error=f"{type(e).__name__}: {e}")

        threads = [threading.Thread(target=main, args=(r,), name=f"rank{r}", daemon=True) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return ClusterResult(returns, errors, self.log, max(self.transport.clock), self.transport.bytes_sent)


class ClusterReplay(FaultInjector):
    """The faults of a logged run, fed back step by step."""

    def __init__(self, log: EventLog):
        faults = [Fault(e["step"], e["rank"], e["fault"], e.get("amount", 0.0), e.get("peer", -1)) for e in log.of("fault")]
        super().__init__(model="scripted", scripted=faults)
