"""safetensors reader and writer (own implementation: header JSON + raw little-endian blocks).

Reader: single files, sharded checkpoints (``*.safetensors.index.json`` or every ``*.safetensors`` of a
folder), memory-mapped, dtypes F64/F32/F16/BF16/F8_E4M3/F8_E5M2/I64/I32/I16/I8/U8/BOOL. Quantized
checkpoints are read the way the reference reads them: an F8 or I8 tensor with a scale beside it
(``{name}_scale_inv`` or ``{name}_scale``) and an optional ``{name}_zero_point`` becomes
``(w - zero_point) * scale`` in fp32 — one scale per tensor, per row, or per block of rows x columns —
and the scale tensors (and activation scales such as ``.input_scale`` / ``.k_scale``) are left out of
the tensor list. Writer: F32 / F16 / BF16 (+ metadata), optional sharding with an index file.

Reference: SafeTensorsReader / SafeTensorsWriter (src/Idrak/Models/SafeTensors.cs:67,1018; scale
handling :58-65,744-815).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Dict, Iterable, Iterator, Mapping, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_ACTIVATION_SCALES = (".input_scale", ".input_zero_point", ".output_scale", ".k_scale", ".v_scale")


class SafeTensorInfo:
    __slots__ = ("name", "dtype", "shape", "start", "end", "file")

    def __init__(self, name, dtype, shape, start, end, file):
        self.name, self.dtype, self.shape, self.start, self.end, self.file = name, dtype, tuple(shape), start, end, file

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def __repr__(self):
        return f"SafeTensorInfo({self.name!r}, {self.dtype}, {list(self.shape)}, {Path(self.file).name})"


class _File:
    def __init__(self, path: str):
        self.path = path
        self.f = open(path, "rb")
        head = self.f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n > size - 8 or n > 100_000_000:
            raise ValueError(f"{path}: header length {n} does not fit the file")
        self.header = json.loads(self.f.read(n).decode("utf-8"))
        self.data_start = 8 + n
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def close(self):
        if self.mm is not None:
            self.mm.close()
            self.mm = None
        self.f.close()


class SafeTensorsReader:
    """Open with :meth:`open` on a file, an index json or a folder. ``read(name)`` returns a torch tensor."""

    def __init__(self, files: Iterable[str]):
        self._files: Dict[str, _File] = {}
        self._entries: Dict[str, SafeTensorInfo] = {}
        self.metadata: Dict[str, str] = {}
        self.left_out: Dict[str, str] = {}
        self.quantization_scales: Dict[str, str] = {}
        self._scalings: Dict[str, Tuple[SafeTensorInfo, Optional[SafeTensorInfo]]] = {}
        self.bytes_read = 0
        for path in files:
            fobj = _File(path)
            self._files[path] = fobj
            for name, spec in fobj.header.items():
                if name == "__metadata__":
                    self.metadata.update({str(k): str(v) for k, v in spec.items()})
                    continue
                dt = spec["dtype"]
                if dt not in _DTYPES:
                    raise NotImplementedError(f"Tensor '{name}' in {path} has type {dt}; supported: {sorted(_DTYPES)}")
                start, end = spec["data_offsets"]
                info = SafeTensorInfo(name, dt, spec["shape"], fobj.data_start + start, fobj.data_start + end, path)
                if info.end - info.start != info.count * _DTYPES[dt][1]:
                    raise ValueError(f"Tensor '{name}' in {path}: byte range does not match its shape")
                self._entries[name] = info
        self._link_scales()

    # ------------------------------------------------------------------ opening
    @classmethod
    def open(cls, path: str | os.PathLike) -> "SafeTensorsReader":
        p = Path(path)
        if p.is_dir():
            idx = sorted(p.glob("*.safetensors.index.json"))
            if idx:
                return cls.open(idx[0])
            files = sorted(str(f) for f in p.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"no .safetensors files in {p}")
            return cls(files)
        if p.name.endswith(".index.json"):
            index = json.loads(p.read_text())
            files = sorted({str(p.parent / f) for f in index["weight_map"].values()})
            return cls(files)
        return cls([str(p)])

    def close(self):
        for f in self._files.values():
            f.close()
        self._files.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ scale bookkeeping
    def _link_scales(self):
        names = set(self._entries)
        for name in sorted(names):
            if name.endswith(_ACTIVATION_SCALES):
                self.quantization_scales[name] = "activations"
        for name in sorted(names):
            info = self._entries[name]
            if info.dtype not in ("F8_E4M3", "F8_E5M2", "I8"):
                continue
            scale = None
            for suffix in ("_scale_inv", "_scale"):
                cand = name + suffix
                if cand in names and cand not in self.quantization_scales:
                    scale = self._entries[cand]
                    break
            if scale is None:
                if info.dtype == "I8":
                    self.left_out[name] = "int8 tensor without a scale beside it"
                continue
            zero = self._entries.get(name + "_zero_point")
            self._scalings[name] = (scale, zero)
            self.quantization_scales[scale.name] = name
            if zero is not None:
                self.quantization_scales[zero.name] = name

    @property
    def tensors(self) -> Dict[str, SafeTensorInfo]:
        return {k: v for k, v in self._entries.items()
                if k not in self.quantization_scales and k not in self.left_out}

    def keys(self):
        return self.tensors.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries and name not in self.quantization_scales and name not in self.left_out

    # ------------------------------------------------------------------ reading
    def _raw(self, info: SafeTensorInfo) -> torch.Tensor:
        f = self._files[info.file]
        self.bytes_read += info.end - info.start
        if info.count == 0:
            return torch.empty(info.shape, dtype=_DTYPES[info.dtype][0])
        buf = np.frombuffer(f.mm, dtype=np.uint8, count=info.end - info.start, offset=info.start)
        t = torch.from_numpy(buf.copy())       # detach from the mapping: the reader may be closed later
        return t.view(_DTYPES[info.dtype][0]).reshape(info.shape)

    def read_raw(self, name: str) -> torch.Tensor:
        """The tensor as stored (no scale applied)."""
        return self._raw(self._entries[name])

    def read(self, name: str, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The tensor's values; quantized weights come back de-quantized in fp32."""
        info = self._entries[name]
        t = self._raw(info)
        if name in self._scalings:
            scale_info, zero_info = self._scalings[name]
            t = _apply_scale(t.float(), self._raw(scale_info).float(),
                             self._raw(zero_info).float() if zero_info is not None else None, name)
        elif info.dtype in ("F8_E4M3", "F8_E5M2"):
            t = t.float()
        return t.to(dtype) if dtype is not None else t

    def read_float(self, name: str) -> torch.Tensor:
        return self.read(name, torch.float32)

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for name in self.tensors:
            yield name, self.read(name)


def _apply_scale(w: torch.Tensor, scale: torch.Tensor, zero: Optional[torch.Tensor], name: str) -> torch.Tensor:
    def expand(s: torch.Tensor) -> torch.Tensor:
        if s.numel() == 1:
            return s.reshape(())
        if w.dim() >= 2 and s.dim() == 1 and s.shape[0] == w.shape[-2]:
            return s.reshape(*([1] * (w.dim() - 2)), -1, 1)
        if w.dim() >= 2 and s.dim() == w.dim() and s.shape[-1] == 1 and s.shape[-2] == w.shape[-2]:
            return s
        if w.dim() >= 2 and s.dim() == w.dim() and tuple(s.shape[:-2]) == tuple(w.shape[:-2]):
            rows, cols = w.shape[-2], w.shape[-1]
            a, b = s.shape[-2], s.shape[-1]
            br, bc = -(-rows // a), -(-cols // b)          # block sizes (ceil)
            # prefer a power-of-two block when the grid allows it (128 for fine-grained FP8 checkpoints)
            for cand in (128, 64, 32, 16):
                if -(-rows // cand) == a:
                    br = cand
                if -(-cols // cand) == b:
                    bc = cand
            full = s.repeat_interleave(br, dim=-2).repeat_interleave(bc, dim=-1)
            return full[..., :rows, :cols]
        raise ValueError(f"scale of '{name}' has shape {list(s.shape)} that does not fit {list(w.shape)}")

    if zero is not None:
        w = w - expand(zero)
    return w * expand(scale)


# --------------------------------------------------------------------------- writer
def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def save_file(tensors: Mapping[str, torch.Tensor], path: str | os.PathLike, metadata: Optional[Mapping[str, str]] = None,
              dtype: Optional[torch.dtype] = None) -> None:
    """Write one safetensors file. ``dtype`` converts floating tensors on the way out (F32/F16/BF16)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs, off = [], 0
    for name, t in tensors.items():
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        if t.dtype not in _NAMES:
            raise NotImplementedError(f"cannot store dtype {t.dtype}")
        b = _to_bytes(t)
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)


def save_sharded(tensors: Mapping[str, torch.Tensor], folder: str | os.PathLike, max_shard_bytes: int = 5 << 30,
                 metadata: Optional[Mapping[str, str]] = None, dtype: Optional[torch.dtype] = None,
                 stem: str = "model") -> list[str]:
    """Write ``stem-0000i-of-0000n.safetensors`` shards plus ``stem.safetensors.index.json``."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for name, t in tensors.items():
        nb = t.numel() * (torch.empty((), dtype=dtype).element_size() if dtype is not None and t.is_floating_point()
                          else t.element_size())
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = t
        cur_bytes += nb
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        out = folder / f"{stem}.safetensors"
        save_file(shards[0], out, metadata, dtype)
        return [str(out)]
    weight_map, files, total = {}, [], 0
    for i, shard in enumerate(shards):
        fname = f"{stem}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, folder / fname, metadata, dtype)
        files.append(str(folder / fname))
        for name, t in shard.items():
            weight_map[name] = fname
            total += t.numel() * t.element_size()
    (folder / f"{stem}.safetensors.index.json").write_text(
        json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=2))
    return files


def load_file(path: str | os.PathLike) -> Dict[str, torch.Tensor]:
    with SafeTensorsReader.open(path) as r:
        return {k: r.read(k) for k in r.tensors}
