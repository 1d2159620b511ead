"""Liveness of ranks through the rendezvous store: learn that a peer is gone before launching work that waits on it.

Every rank bumps a counter in the store from a small thread; ``check()`` - called between steps - compares the
peers' counters with what it saw ``timeout`` seconds ago and raises ``RankTimeout`` naming the silent rank. A rank
that leaves in order says ``bye`` and the others raise ``RankLeft`` at once. Nothing here touches a GPU, so a dead
peer is found on the host, with no kernel or collective of this rank in flight.

Reference: shared-memory writer liveness and the `bye` frame (src/Idrak.Network/Transports/FramedTransport.cs:335-363),
ClusterOptions.Timeout / SharedMemoryCheck.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

from .sim import RankTimeout


class RankLeft(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} left the run: {reason}")
        self.rank = rank


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.2, timeout: float = 5.0, prefix: str = "idrak/hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._seen: Dict[int, tuple] = {}
        self.store.set(f"{prefix}/{rank}", "0")
        self._thread = threading.Thread(target=self._beat, name="idrak-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        n = 0
        while not self._stop.wait(self.interval):
            n += 1
            try:
                self.store.set(f"{self.prefix}/{self.rank}", str(n))
            except Exception:
                return                      # the store is gone: the run is ending

    def bye(self, reason: str = "finished") -> None:
        """Say that this rank leaves on purpose (call between steps, with nothing in flight)."""
        self._stop.set()
        self.store.set(f"{self.prefix}/{self.rank}", f"bye:{reason}")

    def close(self) -> None:
        self._stop.set()

    def _read(self, r: int) -> Optional[str]:
        try:
            return self.store.get(f"{self.prefix}/{r}").decode()
        except Exception:
            return None

    def check(self, now: Optional[float] = None) -> None:
        now = time.monotonic() if now is None else now
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v is not None and v.startswith("bye:"):
                raise RankLeft(r, v[4:])
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > self.timeout:
                raise RankTimeout(self.rank, r, self.timeout, "heartbeat")

    def wait_all_alive(self, seconds: float = 30.0) -> None:
        """Block until every rank has beaten at least once (start-up)."""
        end = time.monotonic() + seconds
        while time.monotonic() < end:
            if all((self._read(r) or "") != "" for r in range(self.world)):
                return
            time.sleep(0.05)
        missing = [r for r in range(self.world) if not self._read(r)]
        raise RankTimeout(self.rank, missing[0], seconds, "first heartbeat")
