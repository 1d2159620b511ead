"""Devices by name, device providers, and the "deferred" device whose tensors are read from a file on first use.

``Device.parse("cuda:1")`` / ``Device.cpu()`` / ``Device.cuda(n)`` / ``Device.default()`` / ``Device.available()`` give
plain ``torch.device`` values plus what the providers registered; a provider (``DEVICE_PROVIDERS``) turns a device type
into a backend (``core.backend``), so a plug-in can add a device type.

``DeferredTensors`` opens a safetensors file (or a sharded folder) without reading the data; ``tensor(name)`` returns a
``DeferredTensor`` that knows its shape and dtype and reads its bytes only when moved (``to(device)``), straight into
pinned staging and on to the GPU. A model whose parameters are deferred costs no host memory until a layer is used -
what lets a 70 B checkpoint open on a small host and stream layer by layer.

Reference: Device (src/Idrak.Abstraction/Device.cs), DeviceProviders (Devices/DeviceProviders.cs), DeferredTensors
(Devices/DeferredTensors.cs), CreateSeparateBackend (Backend.cs).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, List, Optional

import torch

from .registry import SlotTable


def _default_providers(table: SlotTable) -> None:
    from .backend import CpuBackend, CudaBackend
    table.register("cpu", lambda index=0: CpuBackend(), "fallback")
    table.register("cuda", lambda index=0: CudaBackend(index), "fallback")


DEVICE_PROVIDERS: SlotTable = SlotTable("device providers", _default_providers)


class Device:
    @staticmethod
    def cpu() -> torch.device:
        return torch.device("cpu")

    @staticmethod
    def cuda(index: int = 0) -> torch.device:
        return torch.device("cuda", index)

    @staticmethod
    def parse(text: str) -> torch.device:
        """``cpu``, ``cuda``, ``cuda:1``, ``gpu`` / ``gpu:1`` (alias), ``auto`` (first GPU, else the CPU)."""
        t = text.strip().lower()
        if t in ("auto", "default", ""):
            return Device.default()
        if t.startswith("gpu"):
            t = "cuda" + t[3:]
        kind = t.split(":", 1)[0]
        if kind not in DEVICE_PROVIDERS:
            raise ValueError(f"Device '{text}' is not known. Known: {', '.join(DEVICE_PROVIDERS.keys())}")
        return torch.device(t)

    @staticmethod
    def default() -> torch.device:
        env = os.environ.get("IDRAK_DEVICE")
        if env:
            return Device.parse(env)
        return torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")

    @staticmethod
    def available() -> List[torch.device]:
        out = [torch.device("cpu")]
        if torch.cuda.is_available():
            out += [torch.device("cuda", i) for i in range(torch.cuda.device_count())]
        return out

    @staticmethod
    def backend(device):
        d = torch.device(device)
        return DEVICE_PROVIDERS[d.type](d.index or 0)


# --------------------------------------------------------------------------- deferred tensors
_ST_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
              "BOOL": torch.bool}


class DeferredTensor:
    """Shape and dtype now, bytes on first move."""

    def __init__(self, path: str, offset: int, nbytes: int, shape, dtype: torch.dtype, name: str):
        self.path, self.offset, self.nbytes = path, offset, nbytes
        self.shape, self.dtype, self.name = torch.Size(shape), dtype, name
        self.device = "deferred"

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def to(self, device, dtype: Optional[torch.dtype] = None, staging: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reads the bytes (into ``staging`` pinned memory when given) and returns a real tensor on ``device``."""
        dev = torch.device(device)
        if staging is not None and staging.numel() >= self.nbytes:
            buf = staging[: self.nbytes]
        else:
            buf = torch.empty(self.nbytes, dtype=torch.uint8, pin_memory=dev.type == "cuda" and torch.cuda.is_available())
        with open(self.path, "rb") as f:
            f.seek(self.offset)
            got = f.readinto(memoryview(buf.numpy())) if self.nbytes else 0
        if got != self.nbytes:
            raise IOError(f"{self.path}: tensor '{self.name}' is cut short ({got} of {self.nbytes} bytes)")
        t = buf.view(self.dtype).reshape(self.shape) if self.nbytes else torch.empty(self.shape, dtype=self.dtype)
        out = t.to(dev, non_blocking=True)
        if dev.type == "cuda" and staging is not None:
            torch.cuda.current_stream(dev).synchronize()         # the staging buffer is reused by the caller
        return out.to(dtype) if dtype is not None and dtype != out.dtype else (out.clone() if dev.type == "cpu" else out)

    def __repr__(self):
        return f"DeferredTensor({self.name}, {tuple(self.shape)}, {self.dtype}, {os.path.basename(self.path)})"


class DeferredTensors:
    """The index of a safetensors file or of a folder with ``model.safetensors.index.json``; no tensor data is read."""

    def __init__(self, path: str):
        self.entries: Dict[str, DeferredTensor] = {}
        files: List[str] = []
        if os.path.isdir(path):
            idx = os.path.join(path, "model.safetensors.index.json")
            if os.path.isfile(idx):
                with open(idx) as f:
                    files = sorted({os.path.join(path, v) for v in json.load(f)["weight_map"].values()})
            else:
                files = sorted(os.path.join(path, n) for n in os.listdir(path) if n.endswith(".safetensors"))
        else:
            files = [path]
        if not files:
            raise FileNotFoundError(f"no safetensors file in {path}")
        for fp in files:
            with open(fp, "rb") as f:
                (n,) = struct.unpack("<Q", f.read(8))
                if n > 100 << 20:
                    raise ValueError(f"{fp}: header of {n} bytes is not a safetensors header")
                header = json.loads(f.read(n))
            base = 8 + n
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                dt = _ST_DTYPES.get(meta["dtype"])
                if dt is None:
                    raise ValueError(f"{fp}: tensor '{name}' has the unsupported type {meta['dtype']}")
                lo, hi = meta["data_offsets"]
                self.entries[name] = DeferredTensor(fp, base + lo, hi - lo, meta["shape"], dt, name)

    def names(self) -> List[str]:
        return sorted(self.entries)

    def tensor(self, name: str) -> DeferredTensor:
        try:
            return self.entries[name]
        except KeyError:
            raise KeyError(f"tensor '{name}' is not in the file; known: {', '.join(self.names()[:8])} ...")

    def total_bytes(self) -> int:
        return sum(e.nbytes for e in self.entries.values())

    def materialize(self, names: Iterable[str], device, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        """Move a group of tensors (one layer, say) through one pinned staging buffer sized for the largest."""
        want = [self.tensor(n) for n in names]
        dev = torch.device(device)
        staging = None
        if dev.type == "cuda" and want and torch.cuda.is_available():
            staging = torch.empty(max(e.nbytes for e in want), dtype=torch.uint8, pin_memory=True)
        return {e.name: e.to(dev, dtype, staging) for e in want}

    def load_into(self, module: torch.nn.Module, device, dtype: Optional[torch.dtype] = None, prefix: str = "",
                  strict: bool = True) -> List[str]:
        """Fill a module's parameters and buffers (created on the ``meta`` device or anywhere) from the file, one tensor at
        a time. Returns the names the file did not have."""
        missing = []
        own = dict(module.named_parameters())
        own.update(dict(module.named_buffers()))
        for name, p in own.items():
            e = self.entries.get(prefix + name)
            if e is None:
                missing.append(name)
                continue
            if tuple(e.shape) != tuple(p.shape):
                raise ValueError(f"'{name}': the file holds {tuple(e.shape)}, the module wants {tuple(p.shape)}")
            value = e.to(device, dtype or (p.dtype if p.device.type != "meta" else None))
            owner, leaf = module, name
            while "." in leaf:
                head, leaf = leaf.split(".", 1)
                owner = getattr(owner, head)
            if isinstance(p, torch.nn.Parameter):
                setattr(owner, leaf, torch.nn.Parameter(value, requires_grad=p.requires_grad))
            else:
                owner.register_buffer(leaf, value)
        if strict and missing:
            raise KeyError(f"the file lacks {len(missing)} tensors, first: {missing[:4]}")
        return missing
