"""Loading and saving whole models: Hugging Face folders, single safetensors files, GGUF files, ``.ikm``
packages and PyTorch checkpoints.

    model = load_pretrained("path/to/folder-or-file", device="cuda", dtype=torch.bfloat16)
    save_huggingface(model, "out/")            # config.json + model.safetensors (F32) [+ shards]

Reference: PretrainedModel.Load / SaveHuggingFace / AddAdapters / SaveAdapters
(src/Idrak/Models/PretrainedModel.cs:466,205,1199), GgufModel (src/Idrak/Models/GgufModel.cs),
PyTorchCheckpoint (src/Idrak/Models/PyTorchCheckpoint.cs:25).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Optional

import torch

from ..formats.safetensors import SafeTensorsReader, save_sharded
from .checkpoint import from_hf_tensors, idrak_tensors, load_idrak_tensors, to_hf_tensors
from .decoder import Decoder, build_decoder
from .families import hf_config_from_spec, spec_from_hf_config
from .spec import DecoderSpec


def _finish(model: Decoder, device, dtype) -> Decoder:
    model = model.to(device)
    if dtype is not None:
        model = model.to(dtype)
    return model


def load_pretrained(path: str | os.PathLike, device: str | torch.device = "cpu",
                    dtype: Optional[torch.dtype] = None, adapters: Optional[str] = None) -> Decoder:
    """Build a decoder from ``path`` and load its weights.

    ``path`` may be a Hugging Face folder (``config.json`` + safetensors or ``pytorch_model.bin``), a ``.gguf``
    file, an ``.ikm`` package, or a folder written by this package (``spec.json`` + Idrak-named safetensors).
    ``adapters`` names a PEFT folder to attach afterwards.
    """
    p = Path(path)
    if p.is_file() and p.suffix == ".gguf":
        from ..formats.gguf import GgufFile
        with GgufFile(p) as g:
            spec = g.decoder_spec()
            model = build_decoder(spec)
            load_idrak_tensors(model, g.idrak_tensors(spec), strict=False)
        model.source_style = "llama"
    elif p.is_file() and p.suffix == ".ikm":
        from ..formats import ikm
        with ikm.open_package(p) as pkg:
            model = pkg.build_model()
        model.source_style = "llama"
    else:
        folder = p if p.is_dir() else p.parent
        if (folder / "spec.json").exists():
            spec = DecoderSpec.from_json(json.loads((folder / "spec.json").read_text()))
            model = build_decoder(spec)
            with SafeTensorsReader.open(p if p.is_file() else folder) as r:
                load_idrak_tensors(model, {k: r.read_float(k) for k in r.tensors})
            model.source_style = "idrak"
        else:
            cfg_path = folder / "config.json"
            if not cfg_path.exists():
                raise FileNotFoundError(f"{folder} has neither config.json nor spec.json")
            spec, style = spec_from_hf_config(cfg_path)
            model = build_decoder(spec)
            st = sorted(folder.glob("*.safetensors"))
            if p.is_file() and p.suffix == ".safetensors":
                st = [p]
            if st or list(folder.glob("*.safetensors.index.json")):
                with SafeTensorsReader.open(st[0] if len(st) == 1 else folder) as r:
                    tensors = {k: r.read_float(k) for k in r.tensors}
            else:
                bins = sorted(folder.glob("pytorch_model*.bin")) + sorted(folder.glob("*.pth")) + sorted(folder.glob("*.pt"))
                if not bins:
                    raise FileNotFoundError(f"{folder} holds no weights (safetensors, .bin, .pth)")
                from ..formats.pth import load_checkpoint
                tensors = {}
                for b in bins:
                    tensors.update({k: v.float() for k, v in load_checkpoint(b).items() if torch.is_tensor(v)})
            tensors = {(k[len("language_model."):] if k.startswith("language_model.") else k): v
                       for k, v in tensors.items()}
            load_idrak_tensors(model, from_hf_tensors(spec, tensors, style), strict=False)
            model.source_style = style
    model = _finish(model, device, dtype)
    if adapters:
        from ..adapters.peft import load_adapters
        load_adapters(model, adapters)
        model = _finish(model, device, dtype)
    return model


def save_huggingface(model: Decoder, folder: str | os.PathLike, style: Optional[str] = None,
                     dtype: torch.dtype = torch.float32, max_shard_bytes: int = 5 << 30) -> None:
    """``config.json`` + ``model.safetensors`` in Hugging Face names and orientation."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    style = style or ("gpt2" if model.spec.learned_positions else "llama")
    tensors = {k: v.detach().cpu() for k, v in to_hf_tensors(model, style).items()}
    save_sharded(tensors, folder, max_shard_bytes, metadata={"format": "pt"}, dtype=dtype)
    (folder / "config.json").write_text(json.dumps(hf_config_from_spec(model.spec, style), indent=2))


def save_idrak(model: Decoder, folder: str | os.PathLike, dtype: torch.dtype = torch.float32) -> None:
    """``spec.json`` + ``model.safetensors`` under the reference's own tensor names."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = {k: v.detach().cpu() for k, v in idrak_tensors(model).items()}
    save_sharded(tensors, folder, metadata={"format": "idrak"}, dtype=dtype)
    (folder / "spec.json").write_text(model.spec.dumps())
