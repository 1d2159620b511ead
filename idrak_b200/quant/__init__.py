"""Weight quantisation: packed int8 / int4 weights, the de-quant-fused linear op, whole-model quantisation."""
from __future__ import annotations

import torch

from .weights import (GROUP_SIZE, Int4Weight, Int8Weight, dequantize_bf16, qgemm, qlinear, quantize_weight)

__all__ = ["GROUP_SIZE", "Int4Weight", "Int8Weight", "dequantize_bf16", "qgemm", "qlinear", "quantize_weight",
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
