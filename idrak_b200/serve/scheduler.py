"""Python face of the native continuous-batching scheduler and KV block pool (``csrc/scheduler.cpp``).

The scheduler decides, step by step, which requests to prefill and which sequences to advance by one
token, owns the block tables of the paged KV cache (block size 16 by default), shares full prompt
blocks between requests with an identical prefix, preempts the youngest sequence when blocks run
out, and enforces the queue limit and per-request deadlines.

Reference: the serving contracts (queue limit, timeout: src/Idrak.Abstraction/Serving/EngineModel.cs:181-200) and
KeyValuePages' prefix sharing (src/Idrak.Abstraction/Generation/KeyValuePages.cs:20-34); the reference has no
continuous batching, so this component is where the two designs differ most.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from .. import _native

PREFILL, DECODE = 1, 2
_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, ll, d = C.c_void_p, C.c_int, C.c_longlong, C.c_double
    pi, pll = C.POINTER(C.c_int), C.POINTER(C.c_longlong)
    b = _native.bind
    b("idrak_sched_create", vp, [i, i, i, i, i, i])
    b("idrak_sched_destroy", None, [vp])
    b("idrak_sched_add", i, [vp, ll, pi, i, i, d])
    b("idrak_sched_step", i, [vp, d, pi, pll, i, pll, pi])
    b("idrak_sched_seq_info", i, [vp, ll, pi, pi, pi, pi])
    b("idrak_sched_seq_blocks", i, [vp, ll, pi, i])
    b("idrak_sched_seq_tokens", i, [vp, ll, pi, i])
    b("idrak_sched_commit", i, [vp, ll, i, i])
    b("idrak_sched_abort", i, [vp, ll])
    b("idrak_sched_forget", None, [vp, ll])
    b("idrak_sched_stats", None, [vp, pll])
    _BOUND = True


class QueueFull(RuntimeError):
    """The waiting queue is at its limit (the reference's InferenceQueueFullException)."""


@dataclass
class SeqInfo:
    state: int
    length: int
    computed: int
    cached_prefix: int
    n_blocks: int


class Scheduler:
    def __init__(self, num_blocks: int, block_size: int = 16, max_batch: int = 256,
                 max_prefill_tokens: int = 8192, queue_limit: int = 0, prefix_sharing: bool = False):
        _bind()
        self.lib = _native.lib()
        self.block_size, self.num_blocks, self.max_batch = block_size, num_blocks, max_batch
        self._h = self.lib.idrak_sched_create(num_blocks, block_size, max_batch, max_prefill_tokens, queue_limit,
                                              int(prefix_sharing))
        self._ids = (C.c_longlong * max(max_batch, 1))()
        self._expired = (C.c_longlong * max(max_batch, 1))()

    def close(self):
        if self._h:
            self.lib.idrak_sched_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add(self, seq_id: int, prompt: Sequence[int], max_new_tokens: int, deadline: float = 0.0) -> None:
        arr = (C.c_int * len(prompt))(*prompt)
        rc = self.lib.idrak_sched_add(self._h, seq_id, arr, len(prompt), max_new_tokens, float(deadline))
        if rc == -1:
            raise QueueFull("the request queue is full")
        if rc == -2:
            raise ValueError(f"a request of {len(prompt)} + {max_new_tokens} tokens can never fit the KV cache "
                             f"({self.num_blocks} blocks of {self.block_size})")

    def step(self, now: float) -> Tuple[int, List[int], List[int]]:
        """(kind, sequence ids of the step, ids that expired while waiting)."""
        kind, n_exp = C.c_int(0), C.c_int(0)
        n = self.lib.idrak_sched_step(self._h, float(now), C.byref(kind), self._ids, len(self._ids), self._expired,
                                      C.byref(n_exp))
        return kind.value, [int(self._ids[i]) for i in range(n)], [int(self._expired[i]) for i in range(n_exp.value)]

    def info(self, seq_id: int) -> SeqInfo:
        a, b, c, d = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        st = self.lib.idrak_sched_seq_info(self._h, seq_id, C.byref(a), C.byref(b), C.byref(c), C.byref(d))
        if st < 0:
            raise KeyError(seq_id)
        return SeqInfo(st, a.value, b.value, c.value, d.value)

    def blocks(self, seq_id: int, n: int) -> List[int]:
        arr = (C.c_int * max(n, 1))()
        k = self.lib.idrak_sched_seq_blocks(self._h, seq_id, arr, n)
        return [int(arr[i]) for i in range(max(k, 0))]

    def tokens(self, seq_id: int, n: int) -> List[int]:
        arr = (C.c_int * max(n, 1))()
        k = self.lib.idrak_sched_seq_tokens(self._h, seq_id, arr, n)
        return [int(arr[i]) for i in range(max(k, 0))]

    def commit(self, seq_id: int, token: int, finished: bool) -> bool:
        """Record the sampled token; True when the sequence is done (its blocks are released)."""
        return self.lib.idrak_sched_commit(self._h, seq_id, int(token), int(finished)) == 1

    def abort(self, seq_id: int) -> None:
        self.lib.idrak_sched_abort(self._h, seq_id)

    def forget(self, seq_id: int) -> None:
        self.lib.idrak_sched_forget(self._h, seq_id)

    def stats(self) -> dict:
        s = (C.c_longlong * 8)()
        self.lib.idrak_sched_stats(self._h, s)
        keys = ("free_blocks", "total_blocks", "waiting", "running", "preemptions", "rejected", "prefix_hits",
                "block_size")
        return {k: int(s[i]) for i, k in enumerate(keys)}
