"""Token files for pretraining: a flat little-endian array of ids plus a small JSON record beside it.

``train.bin`` holds the ids; ``train.bin.json`` is ``{"format": "idrak-tokens/1", "type": "uint16",
"tokens": N, "documents": D, "separator": id, "vocabulary": V}``. ``TokenFile`` memory-maps the ids (files
larger than memory work) and cuts windows ``[s, s + length)`` with targets shifted by one.

Reference: TokenFileRecord / TokenFileSource / TokenFileWriter (src/Idrak/Datasets/FileSources.cs:8-120).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Iterable, Optional

import numpy as np
import torch

FORMAT = "idrak-tokens/1"
_TYPES = {"uint8": np.uint8, "uint16": np.uint16, "int32": np.int32, "uint32": np.uint32, "int64": np.int64,
          "int16": np.int16, "uint64": np.uint64}


def parse_type(text: str):
    t = text.strip()
    low = t.lower()
    if low in _TYPES:
        return low
    if len(low) > 1 and low[0] in "ui" and low[1:].isdigit():
        full = ("uint" if low[0] == "u" else "int") + low[1:]
        if full in _TYPES:
            return full
    raise ValueError(f"Token ids are stored in an integer type of whole bytes ({', '.join(sorted(_TYPES))}), "
                     f"not '{text}'.")


def record_path(token_file: str | os.PathLike) -> str:
    return str(token_file) + ".json"


def read_type(token_file) -> Optional[str]:
    rp = record_path(token_file)
    if not os.path.exists(rp):
        return None
    try:
        rec = json.loads(Path(rp).read_text())
    except json.JSONDecodeError as e:
        raise ValueError(f"{rp}: the token file's record is not JSON ({e}).")
    if not isinstance(rec, dict) or rec.get("format") != FORMAT:
        return None
    if not isinstance(rec.get("type"), str):
        raise ValueError(f"{rp}: the record names no \"type\" (one of {', '.join(sorted(_TYPES))}).")
    return parse_type(rec["type"])


def write_tokens(path, ids: Iterable[int] | np.ndarray, vocabulary: int, documents: int = 0,
                 separator: Optional[int] = None, dtype: Optional[str] = None) -> dict:
    arr = np.asarray(ids)
    if dtype is None:
        dtype = "uint16" if vocabulary <= 65536 else "int32"
    dtype = parse_type(dtype)
    arr = arr.astype(_TYPES[dtype])
    arr.astype("<" + arr.dtype.str[1:]).tofile(str(path))
    rec = {"documents": int(documents), "format": FORMAT, "tokens": int(arr.size), "type": dtype,
           "vocabulary": int(vocabulary)}
    if separator is not None:
        rec["separator"] = int(separator)
    Path(record_path(path)).write_text(json.dumps(rec, indent=1, sort_keys=True))
    return rec


class TokenFile:
    """Memory-mapped ids cut into training windows."""

    def __init__(self, path, length: int, stride: Optional[int] = None, dtype: Optional[str] = None):
        self.path = str(path)
        t = read_type(path) or (parse_type(dtype) if dtype else None)
        if t is None:
            raise ValueError(f"{path}: no record beside the file and no id type given")
        self.dtype = t
        self.ids = np.memmap(self.path, dtype=np.dtype(_TYPES[t]).newbyteorder("<"), mode="r")
        self.length = int(length)
        self.stride = int(stride or length)
        n = self.ids.shape[0]
        self.windows = max(0, (n - self.length - 1) // self.stride + 1)
        rp = record_path(path)
        self.record = json.loads(Path(rp).read_text()) if os.path.exists(rp) else {}

    def __len__(self) -> int:
        return self.windows

    def window(self, i: int):
        s = i * self.stride
        chunk = np.asarray(self.ids[s: s + self.length + 1]).astype(np.int64)
        return torch.from_numpy(chunk[:-1].copy()), torch.from_numpy(chunk[1:].copy())

    def batch(self, indices: Iterable[int]):
        xs, ys = zip(*(self.window(int(i)) for i in indices))
        return torch.stack(xs), torch.stack(ys)
