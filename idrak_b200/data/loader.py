"""Datasets and the batch loader.

``DataLoader`` draws one epoch's order from its seed exactly as a single process would, so data parallel ranks that
share the seed see one global order:

* ``shard(rank, world)`` - rank takes positions ``k * world + rank`` of the order; batch ``k`` of every rank together is
  batch ``k`` of one process with batches ``world`` times as large.
* ``step_shares(world, place)`` - for groups whose membership changes between steps: each step's
  ``world * batch_size`` samples are dealt to the ranks taking part (``place()`` returns this rank's place and the
  count, or None to sit the step out); every rank yields one item per step.
* bucketed batching (``bucket_by``) groups samples of similar length to cut padding; ``prefetch`` builds batches on a
  worker thread; ``pin_memory`` makes the host batch ready for an asynchronous copy; ``device`` moves it.

Reference: DataLoader (src/Idrak/Datasets/DataLoader.cs:24-230: Shard :150, StepShares :165, transforms, prefetch),
Dataset.cs, SampleViews.cs.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch


class Dataset:
    """Indexable samples: ``len(ds)`` and ``ds[i] -> (features, target)`` (tensors or anything ``collate`` accepts)."""

    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, index: int):
        raise NotImplementedError

    def split(self, fraction: float, seed: int = 0) -> Tuple["Subset", "Subset"]:
        """Two disjoint random views holding ``fraction`` and ``1 - fraction`` of the samples."""
        order = np.random.default_rng(seed).permutation(len(self))
        cut = int(round(len(self) * fraction))
        return Subset(self, order[:cut]), Subset(self, order[cut:])


class TensorDataset(Dataset):
    def __init__(self, features: torch.Tensor, targets: Optional[torch.Tensor] = None):
        if targets is not None and len(features) != len(targets):
            raise ValueError("features and targets need the same number of rows")
        self.features, self.targets = features, targets

    def __len__(self):
        return len(self.features)

    def __getitem__(self, i):
        return (self.features[i], self.targets[i]) if self.targets is not None else (self.features[i],)


class Subset(Dataset):
    def __init__(self, base: Dataset, indices: Sequence[int]):
        self.base, self.indices = base, np.asarray(indices, np.int64)

    def __len__(self):
        return len(self.indices)

    def __getitem__(self, i):
        return self.base[int(self.indices[i])]


class MappedDataset(Dataset):
    def __init__(self, base: Dataset, fn: Callable):
        self.base, self.fn = base, fn

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.fn(self.base[i])


class TokenWindows(Dataset):
    """Fixed-length windows over a flat token array (a mapped token file): sample ``i`` is
    ``(tokens[i * stride : i * stride + length], the same shifted by one)``."""

    def __init__(self, tokens, length: int, stride: Optional[int] = None):
        self.tokens, self.length, self.stride = tokens, length, stride or length
        self.count = max((len(tokens) - length - 1) // self.stride + 1, 0)

    def __len__(self):
        return self.count

    def __getitem__(self, i):
        at = i * self.stride
        w = torch.as_tensor(np.asarray(self.tokens[at: at + self.length + 1]).astype(np.int64))
        return w[:-1], w[1:]


def collate(samples: List) -> Tuple[torch.Tensor, ...]:
    """Stack per-field; variable-length 1-D fields are right-padded with zeros and a lengths tensor is appended."""
    fields = list(zip(*samples))
    out, ragged = [], None
    for f in fields:
        ts = [torch.as_tensor(v) for v in f]
        if ts[0].dim() >= 1 and len({t.shape[0] for t in ts}) > 1:
            ragged = torch.tensor([t.shape[0] for t in ts])
            out.append(torch.nn.utils.rnn.pad_sequence(ts, batch_first=True))
        else:
            out.append(torch.stack(ts))
    if ragged is not None:
        out.append(ragged)
    return tuple(out)


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 32, shuffle: bool = False, drop_last: bool = False,
                 seed: Optional[int] = None, transforms: Sequence[Callable] = (), collate_fn: Callable = collate,
                 bucket_by: Optional[Callable[[int], int]] = None, bucket_size: int = 50, prefetch: int = 0,
                 pin_memory: bool = False, device: Optional[torch.device] = None):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self.seed = 0 if seed is None else seed
        self.transforms, self.collate_fn = list(transforms), collate_fn
        self.bucket_by, self.bucket_size = bucket_by, bucket_size
        self.prefetch, self.pin_memory, self.device = prefetch, pin_memory, device
        self.epoch = 0

    # ------------------------------------------------------------------ order
    def order(self, epoch: int) -> np.ndarray:
        n = len(self.dataset)
        order = np.random.default_rng([self.seed, epoch]).permutation(n) if self.shuffle else np.arange(n)
        if self.bucket_by is not None:
            # sort by length inside windows of bucket_size batches: neighbours in a batch have similar lengths, the
            # windows keep the epoch shuffled at large
            window = self.bucket_size * self.batch_size
            parts = [order[i: i + window] for i in range(0, n, window)]
            order = np.concatenate([p[np.argsort([self.bucket_by(int(j)) for j in p], kind="stable")] for p in parts]) if parts else order
        return order

    def batch_count(self, world: int = 1) -> int:
        per = self.batch_size * world
        n = len(self.dataset)
        return n // per if self.drop_last else (n + per - 1) // per

    def __len__(self) -> int:
        return self.batch_count()

    # ------------------------------------------------------------------ batches
    def _make(self, indices: Iterable[int], epoch: int):
        samples = []
        for i in indices:
            s = self.dataset[int(i)]
            for t in self.transforms:
                s = t(s, epoch, int(i)) if _wants_context(t) else t(s)
            samples.append(s)
        batch = self.collate_fn(samples)
        if self.pin_memory and torch.cuda.is_available():
            batch = tuple(b.pin_memory() if isinstance(b, torch.Tensor) else b for b in batch)
        if self.device is not None:
            batch = tuple(b.to(self.device, non_blocking=True) if isinstance(b, torch.Tensor) else b for b in batch)
        return batch

    def _batches(self, rank: int, world: int) -> Iterator:
        epoch = self.epoch
        self.epoch += 1
        order = self.order(epoch)
        per = self.batch_size * world
        for k in range(self.batch_count(world)):
            step = order[k * per: (k + 1) * per]
            mine = step[rank::world]
            if len(mine):
                yield self._make(mine, epoch)

    def _prefetched(self, it: Iterator) -> Iterator:
        if self.prefetch <= 0:
            yield from it
            return
        q: "queue.Queue" = queue.Queue(maxsize=self.prefetch)
        done, failed = object(), []

        def work():
            try:
                for b in it:
                    q.put(b)
            except BaseException as e:          # surfaced on the consumer's side
                failed.append(e)
            finally:
                q.put(done)

        t = threading.Thread(target=work, daemon=True, name="idrak-loader")
        t.start()
        while True:
            b = q.get()
            if b is done:
                break
            yield b
        t.join()
        if failed:
            raise failed[0]

    def __iter__(self) -> Iterator:
        return self._prefetched(self._batches(0, 1))

    def shard(self, rank: int, world: int) -> Iterator:
        if not 0 <= rank < world:
            raise ValueError("0 <= rank < world")
        return self._prefetched(self._batches(rank, world))

    def step_shares(self, world: int, place: Callable[[], Optional[Tuple[int, int]]]) -> Iterator:
        """One item per step on every rank: this rank's batch, or None when it sits the step out or the step's last
        samples went to the others."""
        if world <= 0:
            raise ValueError("world must be positive")
        epoch = self.epoch
        self.epoch += 1
        order = self.order(epoch)
        per = self.batch_size * world
        for k in range(self.batch_count(world)):
            mine = place()
            if mine is None or mine[1] <= 0:
                yield None
                continue
            step = order[k * per: (k + 1) * per]
            take = step[mine[0]:: mine[1]]
            yield self._make(take, epoch) if len(take) else None


def _wants_context(fn: Callable) -> bool:
    try:
        import inspect
        return len(inspect.signature(fn).parameters) >= 3
    except (TypeError, ValueError):
        return False
