"""Weight quantisation: packed int8 / int4 weights, the de-quant-fused linear op, whole-model quantisation."""
from __future__ import annotations

import torch

from .weights import (GROUP_SIZE, Fp8Weight, Int4Weight, Int8Weight, dequantize_bf16, qgemm, qlinear, quantize_weight)

__all__ = ["GROUP_SIZE", "Fp8Weight", "Int4Weight", "Int8Weight", "dequantize_bf16", "qgemm", "qlinear", "quantize_weight",
           "quantize_model", "dense_weight"]


def dense_weight(owner, name: str) -> torch.Tensor:
    """The ``[out, in]`` matrix of projection ``name`` ("qkv", "o", "up", "down") of an attention or
    feed-forward module, de-quantised when the module holds it packed."""
    w = getattr(owner, f"{name}_weight")
    if w is not None:
        return w
    return owner.packed[name].dequantize().t()


@torch.no_grad()
def quantize_model(model, kind: str = "int8", keep_dense: bool = False):
    """Replace every projection matrix of every block (q/k/v, o, gate/up, down) by a packed weight.

    The dense parameters are dropped (set to ``None``) unless ``keep_dense``; embeddings, norms, biases and
    the head stay as they are. The frozen base of a LoRA / DoRA fine-tune is quantised this way
    (ModuleExtensions.QuantizeInt8 / QuantizeInt4 in the reference, src/Idrak/Layers/ModuleExtensions.cs).
    """
    from ..models.decoder import FeedForward
    n = 0
    for blk in model.blocks:
        owners = [(blk.attn, ("qkv", "o"))]
        if isinstance(blk.mlp, FeedForward):
            owners.append((blk.mlp, ("up", "down")))
        else:
            for e in blk.mlp.experts:
                owners.append((e, ("up", "down")))
            if blk.mlp.shared is not None:
                owners.append((blk.mlp.shared, ("up", "down")))
        for owner, names in owners:
            packed = dict(getattr(owner, "packed", {}))
            for name in names:
                w = getattr(owner, f"{name}_weight")
                if w is None:
                    continue
                packed[name] = quantize_weight(w.detach().t().contiguous(), kind)      # [in, out]
                if not keep_dense:
                    setattr(owner, f"{name}_weight", None)
                n += 1
            owner.packed = packed
    model.quantization = kind
    return n


def _packed_owners(model):
    from ..models.decoder import FeedForward
    for li, blk in enumerate(model.blocks):
        yield f"blocks.{li}.attn", blk.attn
        if isinstance(blk.mlp, FeedForward):
            yield f"blocks.{li}.mlp", blk.mlp
        else:
            for ei, e in enumerate(blk.mlp.experts):
                yield f"blocks.{li}.mlp.experts.{ei}", e
            if blk.mlp.shared is not None:
                yield f"blocks.{li}.mlp.shared", blk.mlp.shared


def save_packed(model, folder) -> None:
    """A quantised model as a folder: ``spec.json``, ``quantization.json`` and ``model.safetensors`` holding the
    packed codes and scales as stored (``<owner>.<name>.codes`` / ``.scales``) beside the dense tensors that stayed
    (embeddings, norms, biases, head)."""
    import json
    from pathlib import Path

    import torch

    from ..formats.safetensors import save_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors, packed_index = {}, {}
    for prefix, owner in _packed_owners(model):
        for name, w in getattr(owner, "packed", {}).items():
            key = f"{prefix}.{name}"
            tensors[key + ".codes"] = w.codes.detach().cpu().contiguous()
            tensors[key + ".scales"] = w.scales.detach().cpu().contiguous()
            packed_index[key] = {"bits": w.bits, "rows": w.rows, "cols": w.cols, "kind": getattr(w, "kind", "int")}
    for n, p in model.named_parameters():
        if p is not None and "adapters" not in n:
            tensors[n] = p.detach().cpu().contiguous()
    save_file(tensors, folder / "model.safetensors", metadata={"format": "idrak-packed"})
    (folder / "spec.json").write_text(model.spec.dumps())
    (folder / "quantization.json").write_text(json.dumps({"kind": getattr(model, "quantization", None),
                                                           "packed": packed_index}, indent=1))


def load_packed(folder, device="cuda"):
    """The model written by ``save_packed``, with its projections still packed."""
    import json
    from pathlib import Path

    import torch

    from ..formats.safetensors import load_file
    from ..models.decoder import build_decoder
    from ..models.spec import DecoderSpec
    from .weights import Fp8Weight, Int4Weight, Int8Weight
    folder = Path(folder)
    spec = DecoderSpec.from_json((folder / "spec.json").read_text())
    info = json.loads((folder / "quantization.json").read_text())
    tensors = load_file(folder / "model.safetensors")
    model = build_decoder(spec).to(device, torch.bfloat16)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n in tensors:
                p.copy_(tensors[n].to(device))
    owners = dict(_packed_owners(model))
    for key, meta in info["packed"].items():
        prefix, name = key.rsplit(".", 1)
        owner = owners[prefix]
        cls = Fp8Weight if meta.get("kind") == "fp8" else (Int4Weight if meta["bits"] == 4 else Int8Weight)
        w = cls(tensors[key + ".codes"].to(device), tensors[key + ".scales"].to(device), meta["rows"], meta["cols"])
        packed = dict(getattr(owner, "packed", {}))
        packed[name] = w
        owner.packed = packed
        setattr(owner, f"{name}_weight", None)
    model.quantization = info.get("kind")
    return model
