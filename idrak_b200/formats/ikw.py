"""``.ikw`` module weight files (IKW2 .. IKW5), reader and writer.

Layout (little-endian): u32 magic ``IKW2``..``IKW5``; for IKW3+ the list of linear-layer positions stored
as int8, for IKW4+ the list stored as bfloat16, for IKW5 the list stored as int4 and the list of
embedding positions stored as bfloat16 (each list: i32 count, i32 positions); then i32 tensor count and
per tensor: i32 rank, i32 dims, (IKW3+) one byte ``WeightFormat`` {0 float32, 1 float16, 2 bfloat16},
raw values. Packed weights (words and scales) are written verbatim as float32-typed words, so they
survive byte for byte. Parameters come first, buffers after, in the module's stable traversal order;
the architecture must match on load (count and every shape are checked).

Reference: ModuleFiles (src/Idrak/ModuleFiles.cs:20-23 magics, :43-111 save, :138-239 load).
"""
from __future__ import annotations

import io
import struct
from dataclasses import dataclass, field
from typing import BinaryIO, List, Sequence

import numpy as np
import torch

MAGIC2, MAGIC3, MAGIC4, MAGIC5 = 0x32574B49, 0x33574B49, 0x34574B49, 0x35574B49
FLOAT32, FLOAT16, BFLOAT16 = 0, 1, 2
_FORMAT_NAMES = {"float32": FLOAT32, "float16": FLOAT16, "bfloat16": BFLOAT16}


@dataclass
class IkwContents:
    version: int
    tensors: List[torch.Tensor]                       # fp32 values (packed words keep their bit patterns)
    formats: List[int] = field(default_factory=list)  # WeightFormat each tensor was stored in
    int8_layers: List[int] = field(default_factory=list)
    bfloat16_layers: List[int] = field(default_factory=list)
    int4_layers: List[int] = field(default_factory=list)
    bfloat16_embeddings: List[int] = field(default_factory=list)


def _read_exact(f: BinaryIO, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise ValueError("unexpected end of .ikw file")
    return b


def _read_i32(f: BinaryIO) -> int:
    return struct.unpack("<i", _read_exact(f, 4))[0]


def _read_list(f: BinaryIO) -> List[int]:
    n = _read_i32(f)
    if n < 0 or n > 1_000_000:
        raise ValueError(f"bad list length {n} in .ikw file")
    return [_read_i32(f) for _ in range(n)]


def read(path_or_file) -> IkwContents:
    """Read every tensor of an ``.ikw`` file as fp32 (float16 / bfloat16 values are widened)."""
    own = isinstance(path_or_file, (str, bytes)) or hasattr(path_or_file, "__fspath__")
    f = open(path_or_file, "rb") if own else path_or_file
    try:
        (magic,) = struct.unpack("<I", _read_exact(f, 4))
        if magic not in (MAGIC2, MAGIC3, MAGIC4, MAGIC5):
            raise ValueError(f"not an .ikw file (magic {magic:#010x})")
        version = {MAGIC2: 2, MAGIC3: 3, MAGIC4: 4, MAGIC5: 5}[magic]
        out = IkwContents(version, [])
        if version >= 3:
            out.int8_layers = _read_list(f)
        if version >= 4:
            out.bfloat16_layers = _read_list(f)
        if version >= 5:
            out.int4_layers = _read_list(f)
            out.bfloat16_embeddings = _read_list(f)
        count = _read_i32(f)
        for _ in range(count):
            rank = _read_i32(f)
            if rank < 0 or rank > 8:
                raise ValueError(f"bad tensor rank {rank}")
            shape = [_read_i32(f) for _ in range(rank)]
            n = int(np.prod(shape)) if shape else 1
            fmt = _read_exact(f, 1)[0] if version >= 3 else FLOAT32
            if fmt == FLOAT32:
                t = torch.from_numpy(np.frombuffer(_read_exact(f, 4 * n), dtype="<f4").copy())
            elif fmt == FLOAT16:
                t = torch.from_numpy(np.frombuffer(_read_exact(f, 2 * n), dtype="<f2").copy()).float()
            elif fmt == BFLOAT16:
                raw = torch.from_numpy(np.frombuffer(_read_exact(f, 2 * n), dtype="<i2").copy())
                t = raw.view(torch.bfloat16).float()
            else:
                raise ValueError(f"unknown WeightFormat {fmt}")
            out.tensors.append(t.reshape(shape))
            out.formats.append(fmt)
        return out
    finally:
        if own:
            f.close()


def write(path_or_file, tensors: Sequence[torch.Tensor], weight_format: int | str = FLOAT32,
          exact: Sequence[bool] | None = None, int8_layers: Sequence[int] = (), bfloat16_layers: Sequence[int] = (),
          int4_layers: Sequence[int] = (), bfloat16_embeddings: Sequence[int] = (), version: int | None = None):
    """Write tensors in order. ``exact[i]`` forces float32 for tensor i (packed words and scales).

    The version is the lowest one that can express the lists given (IKW3 at least, as the reference writes);
    ``version=2`` writes the legacy all-float32 layout.
    """
    if isinstance(weight_format, str):
        weight_format = _FORMAT_NAMES[weight_format]
    five = bool(int4_layers) or bool(bfloat16_embeddings)
    if version is None:
        version = 5 if five else 4 if bfloat16_layers else 3
    own = isinstance(path_or_file, (str, bytes)) or hasattr(path_or_file, "__fspath__")
    f = open(path_or_file, "wb") if own else path_or_file
    try:
        f.write(struct.pack("<I", {2: MAGIC2, 3: MAGIC3, 4: MAGIC4, 5: MAGIC5}[version]))

        def put_list(xs):
            f.write(struct.pack("<i", len(xs)))
            for x in xs:
                f.write(struct.pack("<i", int(x)))

        if version >= 3:
            put_list(int8_layers)
        if version >= 4:
            put_list(bfloat16_layers)
        if version >= 5:
            put_list(int4_layers)
            put_list(bfloat16_embeddings)
        f.write(struct.pack("<i", len(tensors)))
        for i, t in enumerate(tensors):
            t = t.detach().cpu()
            f.write(struct.pack("<i", t.dim()))
            for d in t.shape:
                f.write(struct.pack("<i", int(d)))
            fmt = FLOAT32 if (version == 2 or (exact is not None and exact[i])) else weight_format
            if version >= 3:
                f.write(bytes([fmt]))
            if fmt == FLOAT32:
                f.write(t.float().contiguous().numpy().astype("<f4", copy=False).tobytes())
            elif fmt == FLOAT16:
                f.write(t.to(torch.float16).contiguous().numpy().tobytes())
            else:
                f.write(t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes())
    finally:
        if own:
            f.close()


def save_module(module: torch.nn.Module, path, weight_format: int | str = FLOAT32):
    """Every parameter, then every buffer, of ``module`` (in ``checkpoint_tensors`` order when the module
    defines it, i.e. the reference's layout and ``[in, out]`` orientation; else PyTorch traversal order)."""
    from ..models.checkpoint import module_tensors
    items = module_tensors(module)
    write(path, [t for _, t in items], weight_format)


def load_module(module: torch.nn.Module, path) -> None:
    """Read a file written by :func:`save_module` into a module of the same architecture."""
    from ..models.checkpoint import load_module_tensors, module_tensors
    contents = read(path)
    names = [n for n, _ in module_tensors(module)]
    if len(names) != len(contents.tensors):
        raise ValueError(f"The file has {len(contents.tensors)} parameter tensors but the model has {len(names)}.")
    load_module_tensors(module, dict(zip(names, contents.tensors)), strict_shapes=True)


def to_bytes(tensors: Sequence[torch.Tensor], **kw) -> bytes:
    buf = io.BytesIO()
    write(buf, tensors, **kw)
    return buf.getvalue()
