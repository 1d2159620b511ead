"""PyTorch checkpoints (``.pth`` / ``.pt`` / ``pytorch_model.bin``): read with a restricted unpickler.

Only tensors and plain containers are materialised (``torch.load(weights_only=True)``): a checkpoint
that needs arbitrary classes to unpickle is refused rather than executed. Nested ``state_dict`` /
``model`` / ``module`` wrappers are unwrapped and ``module.`` prefixes of DataParallel checkpoints are
dropped.

Reference: PyTorchCheckpoint, a restricted unpickler over the zip layout
(src/Idrak/Models/PyTorchCheckpoint.cs:25).
"""
from __future__ import annotations

import os
from typing import Dict

import torch


def load_checkpoint(path: str | os.PathLike) -> Dict[str, torch.Tensor]:
    obj = torch.load(str(path), map_location="cpu", weights_only=True)
    for key in ("state_dict", "model_state_dict", "model", "module"):
        if isinstance(obj, dict) and key in obj and isinstance(obj[key], dict):
            obj = obj[key]
    if not isinstance(obj, dict):
        raise ValueError(f"{path}: the checkpoint holds a {type(obj).__name__}, not a mapping of tensors")
    out = {}
    for k, v in obj.items():
        if torch.is_tensor(v):
            out[k[len("module."):] if k.startswith("module.") else k] = v
    return out
