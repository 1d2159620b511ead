"""Keyed registries with override policies, used wherever the package lets plug-ins add or replace an implementation
(model families, tokenizer pieces, tool-call formats, engine model kinds, optimizers).

A ``SlotTable`` maps a key to a stack of entries. ``register(key, value, policy)``:
  * ``"fallback"`` - used only while nothing else is registered for the key (first-party defaults),
  * ``"shadow"``   - goes on top and wins until removed; removing it brings the previous entry back.

Reference: SlotTable<K, V> and its FallBack / Shadow policies (src/Idrak.Abstraction/Overrides/SlotTable.cs:41),
LibraryDefaults.Ensure (lazy registration of first-party entries, LibraryDefaults.cs:18-30).
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, Generic, Iterator, List, Optional, Tuple, TypeVar

K = TypeVar("K")
V = TypeVar("V")


class Slot(Generic[V]):
    def __init__(self, table: "SlotTable", key, value: V, policy: str):
        self.table, self.key, self.value, self.policy = table, key, value, policy

    def remove(self) -> None:
        self.table._remove(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()


class SlotTable(Generic[K, V]):
    def __init__(self, name: str, defaults: Optional[Callable[["SlotTable"], None]] = None):
        self.name = name
        self._slots: Dict[K, List[Slot]] = {}
        self._lock = threading.RLock()
        self._defaults, self._ensured = defaults, defaults is None

    def _ensure(self) -> None:
        if not self._ensured:
            with self._lock:
                if not self._ensured:
                    self._ensured = True
                    self._defaults(self)

    def register(self, key: K, value: V, policy: str = "shadow") -> Slot:
        if policy not in ("shadow", "fallback"):
            raise ValueError("policy must be 'shadow' or 'fallback'")
        slot = Slot(self, key, value, policy)
        with self._lock:
            stack = self._slots.setdefault(key, [])
            if policy == "fallback":
                stack.insert(0, slot)            # below everything registered so far
            else:
                stack.append(slot)
        return slot

    def _remove(self, slot: Slot) -> None:
        with self._lock:
            stack = self._slots.get(slot.key, [])
            if slot in stack:
                stack.remove(slot)
            if not stack:
                self._slots.pop(slot.key, None)

    def get(self, key: K, default: Optional[V] = None) -> Optional[V]:
        self._ensure()
        with self._lock:
            stack = self._slots.get(key)
            return stack[-1].value if stack else default

    def __getitem__(self, key: K) -> V:
        v = self.get(key)
        if v is None:
            raise KeyError(f"{self.name}: nothing registered for '{key}'; known: {', '.join(map(str, self.keys()))}")
        return v

    def __contains__(self, key) -> bool:
        self._ensure()
        return key in self._slots

    def keys(self) -> List[K]:
        self._ensure()
        with self._lock:
            return sorted(self._slots, key=str)

    def items(self) -> Iterator[Tuple[K, V]]:
        for k in self.keys():
            yield k, self.get(k)
