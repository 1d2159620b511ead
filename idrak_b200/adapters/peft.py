"""PEFT adapter folders: ``adapter_config.json`` + ``adapter_model.safetensors``.

Tensor names: ``base_model.model.<checkpoint module path>.lora_A.weight`` ``[r, in]``,
``.lora_B.weight`` ``[out, r]`` and, for DoRA, ``.lora_magnitude_vector`` ``[out]`` — values in F32 with
metadata ``{"format": "pt"}``. The module path is the Hugging Face one
(``model.layers.3.self_attn.q_proj``). The reader accepts only ``peft_type`` LORA, computes the scale as
``alpha / r`` (``alpha / sqrt(r)`` with ``use_rslora``), accepts the ``.default`` infix PEFT writes, and
refuses by name what it does not implement: ``rank_pattern``, ``alpha_pattern``, ``bias`` other than
``none``, ``lora_bias``, ``layer_replication``, ``trainable_token_indices``, ``use_qalora``,
``modules_to_save``. A magnitude vector without ``use_dora`` (or the reverse) is an error.

Reference: PeftAdapterConfig (src/Idrak/Models/PeftAdapters.cs:13-135), PretrainedModel.SaveAdapters
(src/Idrak/Models/PretrainedModel.cs:205,1321-1393), AdapterMerge (PeftAdapters.cs:179).
"""
from __future__ import annotations

import json
import math
import os
from pathlib import Path
from typing import Dict, Optional

import torch

from ..formats.safetensors import SafeTensorsReader, save_file
from ..models.decoder import Decoder
from .lora import DoraAdapter, LoraAdapter, add_adapters, named_adapters

_HF_TARGET = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "gate": "gate_proj", "up": "up_proj",
              "down": "down_proj", "head": "lm_head"}
_FROM_HF = {v: k for k, v in _HF_TARGET.items()}


def hf_module_path(idrak_path: str) -> str:
    """``layers.3.attn.q`` -> ``model.layers.3.self_attn.q_proj``; ``head`` -> ``lm_head``."""
    if idrak_path == "head":
        return "lm_head"
    parts = idrak_path.split(".")
    layer, owner, target = parts[1], parts[2], parts[3]
    return f"model.layers.{layer}.{'self_attn' if owner == 'attn' else 'mlp'}.{_HF_TARGET[target]}"


class PeftConfigError(ValueError):
    pass


def read_config(folder: str | os.PathLike) -> dict:
    path = Path(folder) / "adapter_config.json"
    cfg = json.loads(path.read_text())
    if not isinstance(cfg, dict):
        raise PeftConfigError(f"{path} is not a JSON object.")
    ptype = cfg.get("peft_type")
    if ptype is not None and str(ptype).upper() != "LORA":
        raise NotImplementedError(f"{path}: peft_type \"{ptype}\" is not supported; LoRA adapters are loaded "
                                  "(peft_type LORA, with use_dora for DoRA).")
    if cfg.get("r") is None:
        raise PeftConfigError(f"{path} has no r.")
    rank = int(cfg["r"])
    if rank <= 0:
        raise PeftConfigError(f"{path}: r is {rank}.")
    unsupported = []
    if isinstance(cfg.get("rank_pattern"), dict) and cfg["rank_pattern"]:
        unsupported.append("rank_pattern (ranks per module)")
    if isinstance(cfg.get("alpha_pattern"), dict) and cfg["alpha_pattern"]:
        unsupported.append("alpha_pattern (alphas per module)")
    if cfg.get("bias") not in (None, "none"):
        unsupported.append(f"bias \"{cfg['bias']}\" (trained biases)")
    if cfg.get("lora_bias") is True:
        unsupported.append("lora_bias")
    if isinstance(cfg.get("layer_replication"), list) and cfg["layer_replication"]:
        unsupported.append("layer_replication")
    if cfg.get("trainable_token_indices") is not None:
        unsupported.append("trainable_token_indices")
    if cfg.get("use_qalora") is True:
        unsupported.append("use_qalora")
    if isinstance(cfg.get("modules_to_save"), list) and cfg["modules_to_save"]:
        unsupported.append(f"modules_to_save ({', '.join(map(str, cfg['modules_to_save']))})")
    if unsupported:
        verb = "is" if len(unsupported) == 1 else "are"
        raise NotImplementedError(f"{path}: {', '.join(unsupported)} {verb} not supported; LoRA and DoRA adapters "
                                  "with one rank and alpha for every module are loaded.")
    alpha = float(cfg.get("lora_alpha", rank))
    rslora = cfg.get("use_rslora") is True
    return {"r": rank, "lora_alpha": alpha, "use_rslora": rslora, "use_dora": cfg.get("use_dora") is True,
            "scale": alpha / math.sqrt(rank) if rslora else alpha / rank,
            "target_modules": cfg.get("target_modules") or [], "raw": cfg}


def save_adapters(model: Decoder, folder: str | os.PathLike, base_model_name_or_path: str = "") -> None:
    """Write the model's adapters as a PEFT folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = getattr(model, "adapter_config", None)
    if cfg is None:
        raise ValueError("the model has no adapters")
    tensors: Dict[str, torch.Tensor] = {}
    targets = set()
    for path, ad in named_adapters(model):
        prefix = "base_model.model." + hf_module_path(path)
        tensors[f"{prefix}.lora_A.weight"] = ad.A.detach().float().cpu().contiguous()
        tensors[f"{prefix}.lora_B.weight"] = ad.B.detach().float().cpu().contiguous()
        if isinstance(ad, DoraAdapter):
            tensors[f"{prefix}.lora_magnitude_vector"] = ad.magnitude.detach().float().cpu().contiguous()
        targets.add(hf_module_path(path).split(".")[-1])
    save_file(tensors, folder / "adapter_model.safetensors", metadata={"format": "pt"})
    config = {
        "peft_type": "LORA", "task_type": "CAUSAL_LM", "r": int(cfg["r"]), "lora_alpha": float(cfg["lora_alpha"]),
        "lora_dropout": 0.0, "bias": "none", "fan_in_fan_out": False, "inference_mode": True,
        "use_dora": bool(cfg.get("use_dora", False)), "use_rslora": bool(cfg.get("use_rslora", False)),
        "target_modules": sorted(targets), "base_model_name_or_path": base_model_name_or_path,
    }
    (folder / "adapter_config.json").write_text(json.dumps(config, indent=2))


def load_adapters(model: Decoder, folder: str | os.PathLike) -> dict:
    """Attach the adapters of a PEFT folder to ``model`` (creating them) and load their values."""
    cfg = read_config(folder)
    path = Path(folder) / "adapter_model.safetensors"
    with SafeTensorsReader.open(path) as reader:
        def find(*names) -> Optional[str]:
            for n in names:
                if n in reader:
                    return n
            return None

        present = set()
        for name in reader.keys():
            if ".lora_A" in name:
                mod = name.split(".lora_A")[0]
                leaf = mod.split(".")[-1]
                if leaf not in _FROM_HF:
                    raise NotImplementedError(f"The adapter targets '{mod}', which this decoder has no projection for.")
                present.add(_FROM_HF[leaf])
        add_adapters(model, rank=cfg["r"], alpha=cfg["lora_alpha"], targets=tuple(sorted(present)),
                     dora=cfg["use_dora"], rslora=cfg["use_rslora"])
        loaded = 0
        with torch.no_grad():
            for ipath, ad in named_adapters(model):
                prefix = "base_model.model." + hf_module_path(ipath)
                a = find(f"{prefix}.lora_A.weight", f"{prefix}.lora_A.default.weight")
                if a is None:
                    # a module the adapter does not cover keeps B = 0 (no change to the base)
                    continue
                b = find(f"{prefix}.lora_B.weight", f"{prefix}.lora_B.default.weight")
                if b is None:
                    raise PeftConfigError(f"The adapter has {a} but no lora_B for {hf_module_path(ipath)}.")
                mag = find(f"{prefix}.lora_magnitude_vector", f"{prefix}.lora_magnitude_vector.weight",
                           f"{prefix}.lora_magnitude_vector.default", f"{prefix}.lora_magnitude_vector.default.weight")
                if mag is not None and not cfg["use_dora"]:
                    raise PeftConfigError(f"The adapter has a DoRA magnitude vector for {hf_module_path(ipath)} but "
                                          "its adapter_config.json does not set use_dora.")
                if mag is None and cfg["use_dora"]:
                    raise PeftConfigError(f"The adapter sets use_dora but has no lora_magnitude_vector for "
                                          f"{hf_module_path(ipath)}.")
                ta, tb = reader.read_float(a), reader.read_float(b)
                if tuple(ta.shape) != tuple(ad.A.shape) or tuple(tb.shape) != tuple(ad.B.shape):
                    raise PeftConfigError(f"{hf_module_path(ipath)}: adapter shapes {list(ta.shape)} / "
                                          f"{list(tb.shape)} do not fit the model's {list(ad.A.shape)} / "
                                          f"{list(ad.B.shape)}.")
                ad.A.copy_(ta)
                ad.B.copy_(tb)
                if mag is not None:
                    ad.magnitude.copy_(reader.read_float(mag).reshape(ad.magnitude.shape))
                loaded += 1
    cfg["loaded_modules"] = loaded
    return cfg
