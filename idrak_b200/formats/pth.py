"""PyTorch checkpoints (``.pth`` / ``.pt`` / ``pytorch_model.bin``) read by a restricted unpickler of our own.

A checkpoint written by ``torch.save`` is a zip archive: ``<name>/data.pkl`` (a pickle whose tensors are persistent-id
references ``('storage', storage type, key, location, numel)``) plus one raw file ``<name>/data/<key>`` per storage. The
reader below walks the pickle with an allow-list of exactly the globals a tensor checkpoint needs
(``torch._utils._rebuild_tensor_v2``, the storage type names, ``collections.OrderedDict``, ``torch.Size`` ...): anything
else - a class to instantiate, a function to call - is refused by name, never imported or executed. Storage bytes are read
straight from the archive member (lazily, per tensor). The legacy non-zip format is handed to
``torch.load(weights_only=True)``, which applies the same kind of allow-list.

Nested ``state_dict`` / ``model`` / ``module`` wrappers are unwrapped and ``module.`` prefixes of DataParallel checkpoints
are dropped.

Reference: PyTorchCheckpoint, a restricted unpickler over the zip layout (src/Idrak/Models/PyTorchCheckpoint.cs:25).
"""
from __future__ import annotations

import collections
import os
import pickle
import zipfile
from typing import Any, Dict

import torch

_STORAGE_DTYPES = {
    "FloatStorage": torch.float32, "DoubleStorage": torch.float64, "HalfStorage": torch.float16,
    "BFloat16Storage": torch.bfloat16, "LongStorage": torch.int64, "IntStorage": torch.int32,
    "ShortStorage": torch.int16, "CharStorage": torch.int8, "ByteStorage": torch.uint8, "BoolStorage": torch.bool,
    "Float8_e4m3fnStorage": getattr(torch, "float8_e4m3fn", torch.uint8),
    "Float8_e5m2Storage": getattr(torch, "float8_e5m2", torch.uint8),
}


class UnsafeCheckpoint(pickle.UnpicklingError):
    """The pickle asks for a global outside the allow-list."""


class _StorageType:
    def __init__(self, name: str):
        self.dtype = _STORAGE_DTYPES[name]
        self.name = name


def _rebuild_tensor_v2(storage, storage_offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    t = torch.empty(0, dtype=storage.dtype)
    if len(size) == 0:
        return storage[storage_offset].clone().reshape(())
    return torch.as_strided(storage, tuple(size), tuple(stride), storage_offset)


def _rebuild_parameter(data, requires_grad=False, backward_hooks=None):
    return data


_DTYPE_NAMES = {n: getattr(torch, n) for n in ("float32", "float64", "float16", "bfloat16", "int64", "int32", "int16",
                                               "int8", "uint8", "bool") if hasattr(torch, n)}


class _RestrictedUnpickler(pickle.Unpickler):
    def __init__(self, file, archive: zipfile.ZipFile, prefix: str):
        super().__init__(file)
        self.archive, self.prefix = archive, prefix
        self._storages: Dict[str, torch.Tensor] = {}

    def find_class(self, module: str, name: str) -> Any:
        if module == "collections" and name == "OrderedDict":
            return collections.OrderedDict
        if module == "torch._utils" and name in ("_rebuild_tensor_v2", "_rebuild_tensor"):
            return _rebuild_tensor_v2
        if module == "torch._utils" and name == "_rebuild_parameter":
            return _rebuild_parameter
        if module == "torch" and name in _STORAGE_DTYPES:
            return _StorageType(name)
        if module == "torch" and name == "Size":
            return torch.Size
        if module == "torch" and name in _DTYPE_NAMES:
            return _DTYPE_NAMES[name]
        if module == "torch.serialization" and name == "_get_layout":
            return lambda *_: None
        if module == "builtins" and name in ("set", "frozenset", "dict", "list", "tuple", "int", "float", "str", "bool"):
            return {"set": set, "frozenset": frozenset, "dict": dict, "list": list, "tuple": tuple, "int": int,
                    "float": float, "str": str, "bool": bool}[name]
        raise UnsafeCheckpoint(f"the checkpoint asks for '{module}.{name}', which a tensor checkpoint does not need; refused")

    def persistent_load(self, pid):
        if not isinstance(pid, tuple) or not pid or pid[0] != "storage":
            raise UnsafeCheckpoint(f"unknown persistent id {pid!r}")
        _, kind, key, _location, numel = pid
        dtype = kind.dtype if isinstance(kind, _StorageType) else torch.uint8
        key = str(key)
        if key not in self._storages:
            raw = self.archive.read(f"{self.prefix}/data/{key}")
            item = torch.empty((), dtype=dtype).element_size()
            if len(raw) < int(numel) * item:
                raise pickle.UnpicklingError(f"storage {key} is cut short: {len(raw)} of {int(numel) * item} bytes")
            self._storages[key] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype) if raw else torch.empty(0, dtype=dtype)
        return self._storages[key]


def load_object(path: str | os.PathLike) -> Any:
    """The unpickled object of a zip-format checkpoint through the allow-list; raises ``UnsafeCheckpoint`` otherwise."""
    path = str(path)
    if not zipfile.is_zipfile(path):
        return torch.load(path, map_location="cpu", weights_only=True)          # legacy stream format
    with zipfile.ZipFile(path) as z:
        pkl = [n for n in z.namelist() if n.endswith("/data.pkl") or n == "data.pkl"]
        if not pkl:
            raise ValueError(f"{path}: no data.pkl in the archive (not a torch.save file)")
        prefix = pkl[0][: -len("/data.pkl")] if "/" in pkl[0] else ""
        with z.open(pkl[0]) as f:
            return _RestrictedUnpickler(f, z, prefix).load()


def load_checkpoint(path: str | os.PathLike) -> Dict[str, torch.Tensor]:
    obj = load_object(path)
    for key in ("state_dict", "model_state_dict", "model", "module"):
        if isinstance(obj, dict) and key in obj and isinstance(obj[key], dict):
            obj = obj[key]
    if not isinstance(obj, dict):
        raise ValueError(f"{path}: the checkpoint holds a {type(obj).__name__}, not a mapping of tensors")
    out = {}
    for k, v in obj.items():
        if torch.is_tensor(v):
            out[k[len("module."):] if k.startswith("module.") else k] = v.contiguous()
    return out
