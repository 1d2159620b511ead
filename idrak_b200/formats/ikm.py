"""``.ikm`` model packages: one zip holding a ``manifest.json`` and the entries a served model needs.

Manifest: ``{"format": "idrak-package/1", "created": ISO time, "entries": [{"kind", "name", "file"}]}``.
Entry kinds and their paths: ``Weights`` -> ``weights/NAME.ikw``; ``TrainableWeights`` ->
``trainable/NAME.nsp``; ``Architecture`` -> ``architecture/NAME.json``; ``StandardScaler`` /
``MinMaxScaler`` -> ``scalers/NAME.txt``; ``Tokenizer`` -> ``tokenizers/NAME.json``; ``Json`` ->
``json/NAME.json``; ``Text`` -> ``text/NAME.txt``.

For decoders the ``Architecture`` entry is the ``DecoderSpec`` JSON, so ``reader.build_model()`` rebuilds
the network and loads its weights in one call.

Reference: ModelPackage / ModelPackageWriter / ModelPackageReader
(src/Idrak/Inference/ModelPackage.cs:36-47,152-170,224-231,390-399).
"""
from __future__ import annotations

import datetime as _dt
import io
import json
import os
import struct
import zipfile
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from . import ikw

FORMAT = "idrak-package/1"
DEFAULT_MODEL_NAME = "model"
KINDS = ("Weights", "TrainableWeights", "Architecture", "StandardScaler", "MinMaxScaler", "Tokenizer", "Json", "Text")


@dataclass(frozen=True)
class PackageEntry:
    kind: str
    name: str


def file_name(e: PackageEntry) -> str:
    return {
        "Weights": f"weights/{e.name}.ikw",
        "TrainableWeights": f"trainable/{e.name}.nsp",
        "Architecture": f"architecture/{e.name}.json",
        "StandardScaler": f"scalers/{e.name}.txt",
        "MinMaxScaler": f"scalers/{e.name}.txt",
        "Tokenizer": f"tokenizers/{e.name}.json",
        "Json": f"json/{e.name}.json",
    }.get(e.kind, f"text/{e.name}.txt")


TRAINABLE_MAGIC = 0x31504B49        # "IKP1": selected parameters with their positions


def trainable_to_bytes(module: torch.nn.Module) -> bytes:
    """The parameters that still take gradients, each with its index among ``module.parameters()``:
    u32 magic ``IKP1``, i32 count, then per tensor i32 index, i32 rank, i32 dims, float32 values (little endian).
    Reference: ModuleExtensions.SaveTrainable (src/Idrak/Layers/ModuleExtensions.cs:18,59-83)."""
    chosen = [(i, p) for i, p in enumerate(module.parameters()) if p.requires_grad]
    out = [struct.pack("<Ii", TRAINABLE_MAGIC, len(chosen))]
    for i, p in chosen:
        out.append(struct.pack(f"<ii{p.dim()}i", i, p.dim(), *p.shape))
        out.append(p.detach().to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False).tobytes())
    return b"".join(out)


def load_trainable_bytes(module: torch.nn.Module, data: bytes) -> int:
    """Read what ``trainable_to_bytes`` wrote into the same positions; the index and the shape of every tensor are
    checked against the model. Returns how many tensors were loaded."""
    import numpy as np
    params = list(module.parameters())
    if len(data) < 8 or struct.unpack_from("<I", data, 0)[0] != TRAINABLE_MAGIC:
        raise ValueError("Not a trainable-parameters file (magic IKP1 expected).")
    count = struct.unpack_from("<i", data, 4)[0]
    at = 8
    with torch.no_grad():
        for _ in range(count):
            index, rank = struct.unpack_from("<ii", data, at)
            at += 8
            if index < 0 or index >= len(params):
                raise ValueError(f"The file refers to parameter {index}, but the model has {len(params)}.")
            if rank < 0 or rank > 8:
                raise ValueError(f"Parameter {index}: rank {rank} is not plausible; the file is damaged.")
            shape = struct.unpack_from(f"<{rank}i", data, at)
            at += 4 * rank
            p = params[index]
            if tuple(shape) != tuple(p.shape):
                raise ValueError(f"Parameter {index}: file has {list(shape)}, model has {list(p.shape)}.")
            n = p.numel()
            if at + 4 * n > len(data):
                raise ValueError(f"Parameter {index}: the file ends inside its values.")
            values = np.frombuffer(data, dtype="<f4", count=n, offset=at)
            at += 4 * n
            p.copy_(torch.from_numpy(values.copy()).reshape(p.shape).to(p.dtype))
    return count


class ModelPackageWriter:
    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._entries: List[Tuple[PackageEntry, Callable[[], bytes]]] = []

    def _add(self, kind: str, name: str, producer: Callable[[], bytes]) -> "ModelPackageWriter":
        if kind not in KINDS:
            raise ValueError(f"unknown entry kind '{kind}'")
        if "/" in name or "\\" in name:
            raise ValueError("Entry names cannot contain '/' or '\\'.")
        entry = PackageEntry(kind, name)
        # two entries may not share a path inside the zip (a StandardScaler and a MinMaxScaler of one name would)
        if any(file_name(e) == file_name(entry) for e, _ in self._entries):
            raise ValueError(f"The package already has a {kind} entry named '{name}'.")
        self._entries.append((entry, producer))
        return self

    def weights(self, module: torch.nn.Module, name: str = DEFAULT_MODEL_NAME, weight_format: int | str = ikw.FLOAT32):
        def produce():
            buf = io.BytesIO()
            ikw.save_module(module, buf, weight_format)
            return buf.getvalue()
        return self._add("Weights", name, produce)

    def trainable_weights(self, module: torch.nn.Module, name: str = DEFAULT_MODEL_NAME):
        return self._add("TrainableWeights", name, lambda: trainable_to_bytes(module))

    def architecture(self, description: dict | str, name: str = DEFAULT_MODEL_NAME):
        text = description if isinstance(description, str) else json.dumps(description, indent=2)
        return self._add("Architecture", name, lambda: text.encode("utf-8"))

    def model(self, module: torch.nn.Module, name: str = DEFAULT_MODEL_NAME, weight_format: int | str = ikw.FLOAT32):
        """Weights plus, when the module carries a ``spec``, its architecture."""
        spec = getattr(module, "spec", None)
        if spec is not None:
            self.architecture({"kind": "decoder", "spec": spec.to_json()}, name)
        return self.weights(module, name, weight_format)

    def tokenizer(self, tokenizer_json: dict | str, name: str = DEFAULT_MODEL_NAME):
        text = tokenizer_json if isinstance(tokenizer_json, str) else json.dumps(tokenizer_json)
        return self._add("Tokenizer", name, lambda: text.encode("utf-8"))

    def scaler(self, kind: str, text: str, name: str):
        assert kind in ("StandardScaler", "MinMaxScaler")
        return self._add(kind, name, lambda: text.encode("utf-8"))

    def json(self, document, name: str):
        return self._add("Json", name, lambda: json.dumps(document, indent=2).encode("utf-8"))

    def text(self, text: str, name: str):
        return self._add("Text", name, lambda: text.encode("utf-8"))

    def save(self) -> str:
        manifest = {
            "format": FORMAT,
            "created": _dt.datetime.now(_dt.timezone.utc).isoformat(),
            "entries": [{"kind": e.kind, "name": e.name, "file": file_name(e)} for e, _ in self._entries],
        }
        tmp = self.path + ".tmp"
        with zipfile.ZipFile(tmp, "w", zipfile.ZIP_DEFLATED) as z:
            z.writestr("manifest.json", json.dumps(manifest, indent=2))
            for e, produce in self._entries:
                z.writestr(file_name(e), produce())
        os.replace(tmp, self.path)
        return self.path


class ModelPackageReader:
    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._zip = zipfile.ZipFile(self.path, "r")
        try:
            manifest = json.loads(self._zip.read("manifest.json"))
        except KeyError:
            raise ValueError(f"{self.path}: no manifest.json; not a model package")
        if manifest.get("format") != FORMAT:
            raise ValueError(f"{self.path}: unsupported package format '{manifest.get('format')}'.")
        self.created = manifest.get("created")
        self.entries = [PackageEntry(e["kind"], e["name"]) for e in manifest["entries"]]

    def contains(self, kind: str, name: str = DEFAULT_MODEL_NAME) -> bool:
        return PackageEntry(kind, name) in self.entries

    def _read(self, kind: str, name: str) -> bytes:
        if not self.contains(kind, name):
            raise KeyError(f"{self.path} has no {kind} entry named '{name}'.")
        return self._zip.read(file_name(PackageEntry(kind, name)))

    def load_weights(self, module: torch.nn.Module, name: str = DEFAULT_MODEL_NAME) -> None:
        ikw.load_module(module, io.BytesIO(self._read("Weights", name)))

    def load_trainable(self, module: torch.nn.Module, name: str = DEFAULT_MODEL_NAME) -> None:
        load_trainable_bytes(module, self._read("TrainableWeights", name))

    def architecture(self, name: str = DEFAULT_MODEL_NAME) -> dict:
        return json.loads(self._read("Architecture", name))

    def build_model(self, name: str = DEFAULT_MODEL_NAME, device: str | torch.device = "cpu",
                    dtype: Optional[torch.dtype] = None) -> torch.nn.Module:
        """Rebuild the decoder named ``name`` from its stored spec and load its weights."""
        from ..models import DecoderSpec, build_decoder
        arch = self.architecture(name)
        if arch.get("kind") != "decoder":
            raise ValueError(f"architecture '{name}' is of kind '{arch.get('kind')}', which this build cannot rebuild")
        model = build_decoder(DecoderSpec.from_json(arch["spec"]))
        self.load_weights(model, name)
        model = model.to(device)
        return model.to(dtype) if dtype is not None else model

    def tokenizer(self, name: str = DEFAULT_MODEL_NAME) -> dict:
        return json.loads(self._read("Tokenizer", name))

    def scaler_text(self, name: str) -> str:
        kind = "StandardScaler" if self.contains("StandardScaler", name) else "MinMaxScaler"
        return self._read(kind, name).decode("utf-8")

    def json(self, name: str):
        return json.loads(self._read("Json", name))

    def text(self, name: str) -> str:
        return self._read("Text", name).decode("utf-8")

    def close(self):
        self._zip.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def create(path) -> ModelPackageWriter:
    return ModelPackageWriter(path)


def open_package(path) -> ModelPackageReader:
    return ModelPackageReader(path)
