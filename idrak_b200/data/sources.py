"""Record readers and table operations for building datasets: JSON Lines, JSON, CSV / TSV, plain text, code folders
and Parquet; filter / map / shuffle / dedupe / split / mix over iterables of dict records; CSV tables as feature /
target tensors; feature scalers with the text files the model package stores.

    rows = read_records("train.jsonl")
    rows = dedupe(filter_rows(rows, lambda r: len(r["text"]) > 20), key=lambda r: r["text"])
    train, held = split_rows(list(rows), 0.95, seed=1)

Sources that need the network (hubs, archives over http) are out of reach here and raise by name.

Reference: src/Idrak.Data (DataFiles.cs, DatasetRows.cs, Sources.cs, Parquet/), src/Idrak/Datasets (CsvSource.cs,
Scalers.cs, Deduplication.cs, FileSources.cs).
"""
from __future__ import annotations

import csv
import hashlib
import json
import os
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .loader import TensorDataset

Record = Dict[str, object]
CODE_SUFFIXES = (".py", ".cs", ".ts", ".js", ".java", ".go", ".rs", ".c", ".h", ".cpp", ".hpp", ".cu", ".md")


# ---------------------------------------------------------------------------------------------------------------------
# readers
# ---------------------------------------------------------------------------------------------------------------------
def read_jsonl(path: str) -> Iterator[Record]:
    with open(path, "r", encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                row = json.loads(line)
            except ValueError as e:
                raise ValueError(f"{path}:{n}: not JSON ({e})") from None
            yield row if isinstance(row, dict) else {"value": row}


def read_json(path: str) -> Iterator[Record]:
    with open(path, "r", encoding="utf-8") as f:
        doc = json.load(f)
    rows = doc if isinstance(doc, list) else next((v for v in doc.values() if isinstance(v, list)), [doc])
    for row in rows:
        yield row if isinstance(row, dict) else {"value": row}


def read_delimited(path: str, delimiter: Optional[str] = None) -> Iterator[Record]:
    delimiter = delimiter or ("\t" if path.endswith((".tsv", ".tab")) else ",")
    with open(path, "r", encoding="utf-8", newline="") as f:
        yield from csv.DictReader(f, delimiter=delimiter)


def read_text(path: str, by: str = "line") -> Iterator[Record]:
    """``by``: line (one record per non-empty line), paragraph (blank-line separated) or file."""
    with open(path, "r", encoding="utf-8", errors="replace") as f:
        text = f.read()
    if by == "file":
        yield {"text": text, "source": path}
    elif by == "paragraph":
        for p in text.split("\n\n"):
            if p.strip():
                yield {"text": p.strip(), "source": path}
    elif by == "line":
        for line in text.splitlines():
            if line.strip():
                yield {"text": line, "source": path}
    else:
        raise ValueError("by must be line, paragraph or file")


def read_parquet(path: str, columns: Optional[Sequence[str]] = None) -> Iterator[Record]:
    import pyarrow.parquet as pq
    table = pq.ParquetFile(path)
    for batch in table.iter_batches(columns=list(columns) if columns else None):
        yield from batch.to_pylist()


def read_code(folder: str, suffixes: Sequence[str] = CODE_SUFFIXES, max_bytes: int = 1 << 20) -> Iterator[Record]:
    """One record per source file under ``folder`` (sorted walk, hidden folders skipped)."""
    for root, dirs, files in os.walk(folder):
        dirs[:] = sorted(d for d in dirs if not d.startswith("."))
        for name in sorted(files):
            if name.endswith(tuple(suffixes)):
                p = os.path.join(root, name)
                if os.path.getsize(p) <= max_bytes:
                    with open(p, "r", encoding="utf-8", errors="replace") as f:
                        yield {"text": f.read(), "path": os.path.relpath(p, folder), "language": os.path.splitext(name)[1][1:]}


READERS = {".jsonl": read_jsonl, ".ndjson": read_jsonl, ".json": read_json, ".csv": read_delimited, ".tsv": read_delimited,
           ".txt": read_text, ".md": read_text, ".parquet": read_parquet}


def read_records(source: str, **options) -> Iterator[Record]:
    """Records of a file (by extension) or of every readable file in a folder (sorted)."""
    if source.startswith(("http://", "https://", "hf://", "github://", "kaggle://", "zenodo://")):
        raise OSError(f"'{source}': remote sources need the network, which this machine does not have; copy the file here")
    if os.path.isdir(source):
        for name in sorted(os.listdir(source)):
            p = os.path.join(source, name)
            if os.path.isfile(p) and os.path.splitext(name)[1].lower() in READERS:
                yield from read_records(p, **options)
        return
    ext = os.path.splitext(source)[1].lower()
    if ext not in READERS:
        raise ValueError(f"'{source}': no reader for '{ext}'; known: {', '.join(sorted(READERS))}")
    yield from READERS[ext](source, **options)


def write_jsonl(rows: Iterable[Record], path: str) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n


# ---------------------------------------------------------------------------------------------------------------------
# row operations
# ---------------------------------------------------------------------------------------------------------------------
def filter_rows(rows: Iterable[Record], keep: Callable[[Record], bool]) -> Iterator[Record]:
    return (r for r in rows if keep(r))


def map_rows(rows: Iterable[Record], fn: Callable[[Record], Optional[Record]]) -> Iterator[Record]:
    for r in rows:
        out = fn(r)
        if out is not None:
            yield out


def shuffle_rows(rows: Iterable[Record], seed: int = 0, buffer: int = 0) -> Iterator[Record]:
    """A full shuffle (``buffer = 0``: the rows are held in memory) or a streaming shuffle through a buffer."""
    rng = np.random.default_rng(seed)
    if buffer <= 0:
        rows = list(rows)
        for i in rng.permutation(len(rows)):
            yield rows[int(i)]
        return
    held: List[Record] = []
    for r in rows:
        if len(held) < buffer:
            held.append(r)
            continue
        j = int(rng.integers(0, buffer))
        yield held[j]
        held[j] = r
    for i in rng.permutation(len(held)):
        yield held[int(i)]


def _normalise(text: str) -> str:
    return " ".join(text.lower().split())


def dedupe(rows: Iterable[Record], key: Callable[[Record], str] = lambda r: str(r.get("text", r)),
           near: bool = False, shingle: int = 5, threshold: float = 0.8, bands: int = 16) -> Iterator[Record]:
    """Drop repeats. Exact mode hashes the whitespace- and case-normalised key. ``near=True`` adds MinHash over
    word shingles with banded lookup: a row is dropped when its estimated Jaccard similarity to a kept row reaches
    ``threshold``."""
    seen = set()
    rows_per_band = 4
    n_hash = bands * rows_per_band
    buckets: List[Dict[bytes, List[np.ndarray]]] = [dict() for _ in range(bands)]
    salts = np.random.default_rng(12345).integers(1, 1 << 61, size=n_hash, dtype=np.uint64)
    for r in rows:
        text = _normalise(key(r))
        h = hashlib.blake2b(text.encode("utf-8"), digest_size=16).digest()
        if h in seen:
            continue
        if near:
            words = text.split()
            grams = {" ".join(words[i: i + shingle]) for i in range(max(len(words) - shingle + 1, 1))}
            base = np.array([int.from_bytes(hashlib.blake2b(g.encode("utf-8"), digest_size=8).digest(), "little") for g in grams],
                            dtype=np.uint64)
            with np.errstate(over="ignore"):
                sig = ((base[None, :] ^ salts[:, None]) * np.uint64(0x9E3779B97F4A7C15)).min(axis=1)
            dup = False
            keys = [sig[b * rows_per_band: (b + 1) * rows_per_band].tobytes() for b in range(bands)]
            for b, k in enumerate(keys):
                for other in buckets[b].get(k, ()):
                    if float((other == sig).mean()) >= threshold:
                        dup = True
                        break
                if dup:
                    break
            if dup:
                continue
            for b, k in enumerate(keys):
                buckets[b].setdefault(k, []).append(sig)
        seen.add(h)
        yield r


def split_rows(rows: Sequence[Record], fraction: float, seed: int = 0) -> Tuple[List[Record], List[Record]]:
    order = np.random.default_rng(seed).permutation(len(rows))
    cut = int(round(len(rows) * fraction))
    return [rows[int(i)] for i in order[:cut]], [rows[int(i)] for i in order[cut:]]


def mix(sources: Sequence[Iterable[Record]], weights: Optional[Sequence[float]] = None, seed: int = 0,
        stop: str = "all") -> Iterator[Record]:
    """Interleave sources, drawing the next source by weight. ``stop``: 'all' runs until every source is empty
    (an empty one leaves the draw), 'first' stops when any source ends."""
    its = [iter(s) for s in sources]
    w = np.asarray(weights if weights is not None else [1.0] * len(its), np.float64)
    alive = np.ones(len(its), bool)
    rng = np.random.default_rng(seed)
    while alive.any():
        p = w * alive
        i = int(rng.choice(len(its), p=p / p.sum()))
        try:
            yield next(its[i])
        except StopIteration:
            if stop == "first":
                return
            alive[i] = False


# ---------------------------------------------------------------------------------------------------------------------
# tables and scalers
# ---------------------------------------------------------------------------------------------------------------------
def csv_dataset(path: str, targets: Sequence[str], features: Optional[Sequence[str]] = None,
                delimiter: Optional[str] = None) -> Tuple[TensorDataset, List[str], Dict[str, List[str]]]:
    """Numeric table -> ``TensorDataset(features, targets)``. Text columns become category indices (in order of first
    appearance); the mapping comes back as the third value. Returns (dataset, feature names, categories)."""
    rows = list(read_delimited(path, delimiter))
    if not rows:
        raise ValueError(f"{path}: no rows")
    names = list(rows[0])
    for t in targets:
        if t not in names:
            raise KeyError(f"{path}: no column '{t}'; columns: {', '.join(names)}")
    feats = list(features) if features is not None else [n for n in names if n not in targets]
    cats: Dict[str, List[str]] = {}

    def column(name):
        vals = [r[name] for r in rows]
        try:
            return np.array([float(v) for v in vals], np.float32)
        except (TypeError, ValueError):
            order = cats.setdefault(name, [])
            for v in vals:
                if v not in order:
                    order.append(v)
            return np.array([order.index(v) for v in vals], np.float32)

    x = np.stack([column(n) for n in feats], axis=1)
    y = np.stack([column(n) for n in targets], axis=1)
    return TensorDataset(torch.from_numpy(x), torch.from_numpy(y)), feats, cats


class StandardScaler:
    """Per-column ``(x - mean) / std``; ``save`` / ``load`` use one ``mean std`` pair per line."""

    def __init__(self, mean: Optional[torch.Tensor] = None, std: Optional[torch.Tensor] = None):
        self.mean, self.std = mean, std

    def fit(self, x: torch.Tensor) -> "StandardScaler":
        self.mean = x.float().mean(0)
        std = x.float().std(0, unbiased=False)
        self.std = torch.where(std > 0, std, torch.ones_like(std))
        return self

    def transform(self, x: torch.Tensor) -> torch.Tensor:
        return (x - self.mean.to(x.device)) / self.std.to(x.device)

    def inverse(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.std.to(x.device) + self.mean.to(x.device)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write("standard\n")
            for m, s in zip(self.mean.tolist(), self.std.tolist()):
                f.write(f"{m!r} {s!r}\n")


class MinMaxScaler:
    def __init__(self, low: Optional[torch.Tensor] = None, high: Optional[torch.Tensor] = None):
        self.low, self.high = low, high

    def fit(self, x: torch.Tensor) -> "MinMaxScaler":
        self.low, self.high = x.float().min(0).values, x.float().max(0).values
        return self

    def transform(self, x: torch.Tensor) -> torch.Tensor:
        span = (self.high - self.low).to(x.device)
        return (x - self.low.to(x.device)) / torch.where(span > 0, span, torch.ones_like(span))

    def inverse(self, x: torch.Tensor) -> torch.Tensor:
        return x * (self.high - self.low).to(x.device) + self.low.to(x.device)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write("minmax\n")
            for a, b in zip(self.low.tolist(), self.high.tolist()):
                f.write(f"{a!r} {b!r}\n")


def load_scaler(path: str):
    with open(path, "r", encoding="utf-8") as f:
        kind = f.readline().strip()
        pairs = [tuple(float(v) for v in line.split()) for line in f if line.strip()]
    a = torch.tensor([p[0] for p in pairs], dtype=torch.float32)
    b = torch.tensor([p[1] for p in pairs], dtype=torch.float32)
    if kind == "standard":
        return StandardScaler(a, b)
    if kind == "minmax":
        return MinMaxScaler(a, b)
    raise ValueError(f"{path}: unknown scaler kind '{kind}'")
