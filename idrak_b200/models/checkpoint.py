"""Mapping between the decoder's kernel-friendly parameters and checkpoint layouts.

Two external layouts:

* **Idrak layout** — the reference's names and ``[in, out]`` weight orientation: ``embed.weight``,
  ``pos.weight``, ``layers.i.attn_norm``, ``layers.i.attn.{q,k,v,o}``, ``layers.i.attn.{q,k}_norm``,
  ``layers.i.mlp_norm``, ``layers.i.post_attn_norm``, ``layers.i.post_mlp_norm``,
  ``layers.i.mlp.{gate,up,down}``, MoE ``layers.i.mlp.router`` / ``experts.j.*`` / ``shared.*`` /
  ``shared_gate``, ``norm``, ``head`` (src/Idrak.Abstraction/Generation/DecoderSpec.cs:44-60,
  src/Idrak/Layers/DecoderBuilder.cs:201-412). Used by ``.ikw``, ``.ikm`` and Idrak-style safetensors.
* **Hugging Face layout** — ``model.embed_tokens.weight``, ``model.layers.i.self_attn.q_proj.weight``
  (``[out, in]``) ... for Llama-like families and ``transformer.h.i.attn.c_attn`` ... for GPT-2; the
  reference transposes at this boundary (src/Idrak/Models/PretrainedModel.cs:1358-1360).

The in-memory model keeps one packed QKV matrix and one packed gate/up matrix per block in
``nn.Linear`` orientation; this module splits / joins and transposes at the file boundary, and strips
or restores the padding rows of the vocabulary tables.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

from .decoder import Decoder, FeedForward, MixtureOfExperts
from .spec import DecoderSpec


def _t(w: torch.Tensor) -> torch.Tensor:
    return w.detach().t().contiguous()


def _ff_tensors(prefix: str, ff: FeedForward, spec: DecoderSpec, out: "OrderedDict[str, torch.Tensor]"):
    hidden = ff.down_weight.shape[1]
    if spec.gated:
        out[f"{prefix}.gate.weight"] = _t(ff.up_weight[:hidden])
        if ff.up_bias is not None:
            out[f"{prefix}.gate.bias"] = ff.up_bias[:hidden].detach().clone()
        out[f"{prefix}.up.weight"] = _t(ff.up_weight[hidden:])
        if ff.up_bias is not None:
            out[f"{prefix}.up.bias"] = ff.up_bias[hidden:].detach().clone()
    else:
        out[f"{prefix}.up.weight"] = _t(ff.up_weight)
        if ff.up_bias is not None:
            out[f"{prefix}.up.bias"] = ff.up_bias.detach().clone()
    out[f"{prefix}.down.weight"] = _t(ff.down_weight)
    if ff.down_bias is not None:
        out[f"{prefix}.down.bias"] = ff.down_bias.detach().clone()


def idrak_tensors(model: Decoder) -> "OrderedDict[str, torch.Tensor]":
    """The model's weights under the reference's names, ``[in, out]`` orientation, vocabulary unpadded."""
    spec = model.spec
    V, H, Hkv, D = spec.vocabulary, spec.heads, spec.kv_heads, spec.head_dim
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    out["embed.weight"] = model.embed[:V].detach().clone()
    if model.pos is not None:
        out["pos.weight"] = model.pos.detach().clone()

    def norm(name, n):
        out[f"{name}.weight"] = n.weight.detach().clone()
        if n.bias is not None:
            out[f"{name}.bias"] = n.bias.detach().clone()

    for i, blk in enumerate(model.blocks):
        p = f"layers.{i}"
        norm(f"{p}.attn_norm", blk.attn_norm)
        a = blk.attn
        qw, kw, vw = a.qkv_weight[:H * D], a.qkv_weight[H * D:(H + Hkv) * D], a.qkv_weight[(H + Hkv) * D:]
        for nm, w, lo, hi in (("q", qw, 0, H * D), ("k", kw, H * D, (H + Hkv) * D), ("v", vw, (H + Hkv) * D, None)):
            out[f"{p}.attn.{nm}.weight"] = _t(w)
            if a.qkv_bias is not None:
                out[f"{p}.attn.{nm}.bias"] = a.qkv_bias[lo:hi].detach().clone()
        out[f"{p}.attn.o.weight"] = _t(a.o_weight)
        if a.o_bias is not None:
            out[f"{p}.attn.o.bias"] = a.o_bias.detach().clone()
        if spec.qk_norm:
            out[f"{p}.attn.q_norm.weight"] = a.q_norm.weight.detach().clone()
            out[f"{p}.attn.k_norm.weight"] = a.k_norm.weight.detach().clone()
        if spec.post_norms:
            norm(f"{p}.post_attn_norm", blk.post_attn_norm)
        norm(f"{p}.mlp_norm", blk.mlp_norm)
        if isinstance(blk.mlp, MixtureOfExperts):
            out[f"{p}.mlp.router.weight"] = _t(blk.mlp.router)
            for j, e in enumerate(blk.mlp.experts):
                _ff_tensors(f"{p}.mlp.experts.{j}", e, spec, out)
            if blk.mlp.shared is not None:
                _ff_tensors(f"{p}.mlp.shared", blk.mlp.shared, spec, out)
                out[f"{p}.mlp.shared_gate.weight"] = _t(blk.mlp.shared_gate)
        else:
            _ff_tensors(f"{p}.mlp", blk.mlp, spec, out)
        if spec.post_norms:
            norm(f"{p}.post_mlp_norm", blk.post_mlp_norm)
    norm("norm", model.norm)
    if model.head is not None:
        out["head.weight"] = _t(model.head[:V])
    if model.head_bias is not None:
        out["head.bias"] = model.head_bias[:V].detach().clone()
    return out


def _load_ff(prefix: str, ff: FeedForward, spec: DecoderSpec, src: Mapping[str, torch.Tensor], used: set):
    hidden = ff.down_weight.shape[1]

    def get(name):
        used.add(name)
        return src[name]

    with torch.no_grad():
        if spec.gated:
            ff.up_weight[:hidden].copy_(get(f"{prefix}.gate.weight").t())
            ff.up_weight[hidden:].copy_(get(f"{prefix}.up.weight").t())
            if ff.up_bias is not None:
                ff.up_bias[:hidden].copy_(get(f"{prefix}.gate.bias"))
                ff.up_bias[hidden:].copy_(get(f"{prefix}.up.bias"))
        else:
            ff.up_weight.copy_(get(f"{prefix}.up.weight").t())
            if ff.up_bias is not None:
                ff.up_bias.copy_(get(f"{prefix}.up.bias"))
        ff.down_weight.copy_(get(f"{prefix}.down.weight").t())
        if ff.down_bias is not None:
            ff.down_bias.copy_(get(f"{prefix}.down.bias"))


def load_idrak_tensors(model: Decoder, src: Mapping[str, torch.Tensor], strict: bool = True) -> List[str]:
    """Copy tensors in the reference's layout into the model. Returns the names that were not used."""
    spec = model.spec
    V, H, Hkv, D = spec.vocabulary, spec.heads, spec.kv_heads, spec.head_dim
    used: set = set()

    def get(name):
        if name not in src:
            raise KeyError(f"The weights have no '{name}'.")
        used.add(name)
        return src[name]

    def check(name, t, shape):
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"Shape mismatch for '{name}': file has {list(t.shape)}, model has {list(shape)}.")
        return t

    def norm(name, n):
        n.weight.copy_(check(f"{name}.weight", get(f"{name}.weight"), n.weight.shape))
        if n.bias is not None:
            n.bias.copy_(get(f"{name}.bias"))

    with torch.no_grad():
        model.embed.zero_()
        model.embed[:V].copy_(check("embed.weight", get("embed.weight"), (V, spec.dim)))
        if model.pos is not None:
            model.pos.copy_(check("pos.weight", get("pos.weight"), model.pos.shape))
        for i, blk in enumerate(model.blocks):
            p = f"layers.{i}"
            norm(f"{p}.attn_norm", blk.attn_norm)
            a = blk.attn
            a.qkv_weight[:H * D].copy_(check(f"{p}.attn.q.weight", get(f"{p}.attn.q.weight"), (spec.dim, H * D)).t())
            a.qkv_weight[H * D:(H + Hkv) * D].copy_(
                check(f"{p}.attn.k.weight", get(f"{p}.attn.k.weight"), (spec.dim, Hkv * D)).t())
            a.qkv_weight[(H + Hkv) * D:].copy_(
                check(f"{p}.attn.v.weight", get(f"{p}.attn.v.weight"), (spec.dim, Hkv * D)).t())
            if a.qkv_bias is not None:
                a.qkv_bias[:H * D].copy_(get(f"{p}.attn.q.bias"))
                a.qkv_bias[H * D:(H + Hkv) * D].copy_(get(f"{p}.attn.k.bias"))
                a.qkv_bias[(H + Hkv) * D:].copy_(get(f"{p}.attn.v.bias"))
            a.o_weight.copy_(check(f"{p}.attn.o.weight", get(f"{p}.attn.o.weight"), (H * D, spec.dim)).t())
            if a.o_bias is not None:
                a.o_bias.copy_(get(f"{p}.attn.o.bias"))
            if spec.qk_norm:
                a.q_norm.weight.copy_(get(f"{p}.attn.q_norm.weight"))
                a.k_norm.weight.copy_(get(f"{p}.attn.k_norm.weight"))
            if spec.post_norms:
                norm(f"{p}.post_attn_norm", blk.post_attn_norm)
            norm(f"{p}.mlp_norm", blk.mlp_norm)
            if isinstance(blk.mlp, MixtureOfExperts):
                blk.mlp.router.copy_(get(f"{p}.mlp.router.weight").t())
                for j, e in enumerate(blk.mlp.experts):
                    _load_ff(f"{p}.mlp.experts.{j}", e, spec, src, used)
                if blk.mlp.shared is not None:
                    _load_ff(f"{p}.mlp.shared", blk.mlp.shared, spec, src, used)
                    blk.mlp.shared_gate.copy_(get(f"{p}.mlp.shared_gate.weight").t())
            else:
                _load_ff(f"{p}.mlp", blk.mlp, spec, src, used)
            if spec.post_norms:
                norm(f"{p}.post_mlp_norm", blk.post_mlp_norm)
        norm("norm", model.norm)
        if model.head is not None:
            model.head.zero_()
            model.head[:V].copy_(check("head.weight", get("head.weight"), (spec.dim, V)).t())
        if model.head_bias is not None:
            model.head_bias.zero_()
            model.head_bias[:V].copy_(get("head.bias"))
    unused = [k for k in src if k not in used]
    if strict and unused:
        raise ValueError(f"tensors not used by the model: {unused[:8]}{' ...' if len(unused) > 8 else ''}")
    return unused


# --------------------------------------------------------------------------- generic modules
def module_tensors(module: torch.nn.Module) -> List[Tuple[str, torch.Tensor]]:
    """(name, tensor) pairs a weights file stores for ``module``: the reference's layout for a Decoder,
    parameters then buffers in traversal order for anything else."""
    if isinstance(module, Decoder):
        return list(idrak_tensors(module).items())
    items = [(n, p.detach()) for n, p in module.named_parameters()]
    items += [(n, b.detach()) for n, b in module.named_buffers()]
    return items


def load_module_tensors(module: torch.nn.Module, tensors: Mapping[str, torch.Tensor], strict_shapes: bool = True):
    if isinstance(module, Decoder):
        load_idrak_tensors(module, tensors, strict=True)
        return
    own = dict(module.named_parameters())
    own.update(dict(module.named_buffers()))
    with torch.no_grad():
        for name, t in tensors.items():
            if name not in own:
                raise KeyError(f"The model has no tensor '{name}'.")
            if strict_shapes and tuple(own[name].shape) != tuple(t.shape):
                raise ValueError(f"Shape mismatch: file has {list(t.shape)}, model has {list(own[name].shape)}.")
            own[name].copy_(t.reshape(own[name].shape))


# --------------------------------------------------------------------------- Hugging Face names
def hf_name_map(spec: DecoderSpec, style: str = "llama") -> Dict[str, Tuple[str, bool]]:
    """Idrak name -> (Hugging Face name, transpose?) for the two checkpoint styles this package writes."""
    m: Dict[str, Tuple[str, bool]] = {}
    if style == "gpt2":
        m["embed.weight"] = ("transformer.wte.weight", False)
        m["pos.weight"] = ("transformer.wpe.weight", False)
        for i in range(spec.layers):
            p, h = f"layers.{i}", f"transformer.h.{i}"
            for a, b in (("attn_norm", "ln_1"), ("mlp_norm", "ln_2")):
                m[f"{p}.{a}.weight"] = (f"{h}.{b}.weight", False)
                m[f"{p}.{a}.bias"] = (f"{h}.{b}.bias", False)
            # GPT-2 stores Conv1D weights as [in, out]: no transpose; q, k, v are fused in c_attn
            m[f"{p}.attn.o.weight"] = (f"{h}.attn.c_proj.weight", False)
            m[f"{p}.attn.o.bias"] = (f"{h}.attn.c_proj.bias", False)
            m[f"{p}.mlp.up.weight"] = (f"{h}.mlp.c_fc.weight", False)
            m[f"{p}.mlp.up.bias"] = (f"{h}.mlp.c_fc.bias", False)
            m[f"{p}.mlp.down.weight"] = (f"{h}.mlp.c_proj.weight", False)
            m[f"{p}.mlp.down.bias"] = (f"{h}.mlp.c_proj.bias", False)
        m["norm.weight"] = ("transformer.ln_f.weight", False)
        m["norm.bias"] = ("transformer.ln_f.bias", False)
        return m
    m["embed.weight"] = ("model.embed_tokens.weight", False)
    for i in range(spec.layers):
        p, h = f"layers.{i}", f"model.layers.{i}"
        m[f"{p}.attn_norm.weight"] = (f"{h}.input_layernorm.weight", False)
        m[f"{p}.mlp_norm.weight"] = (f"{h}.post_attention_layernorm.weight", False)
        if spec.post_norms:      # Gemma 2 / 3 naming
            m[f"{p}.post_attn_norm.weight"] = (f"{h}.post_attention_layernorm.weight", False)
            m[f"{p}.mlp_norm.weight"] = (f"{h}.pre_feedforward_layernorm.weight", False)
            m[f"{p}.post_mlp_norm.weight"] = (f"{h}.post_feedforward_layernorm.weight", False)
        for a, b in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "o_proj")):
            m[f"{p}.attn.{a}.weight"] = (f"{h}.self_attn.{b}.weight", True)
            m[f"{p}.attn.{a}.bias"] = (f"{h}.self_attn.{b}.bias", False)
        m[f"{p}.attn.q_norm.weight"] = (f"{h}.self_attn.q_norm.weight", False)
        m[f"{p}.attn.k_norm.weight"] = (f"{h}.self_attn.k_norm.weight", False)
        for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
            m[f"{p}.mlp.{a}.weight"] = (f"{h}.mlp.{b}.weight", True)
            m[f"{p}.mlp.{a}.bias"] = (f"{h}.mlp.{b}.bias", False)
        if spec.experts:
            m[f"{p}.mlp.router.weight"] = (f"{h}.mlp.gate.weight", True)
            for j in range(spec.experts):
                for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                    m[f"{p}.mlp.experts.{j}.{a}.weight"] = (f"{h}.mlp.experts.{j}.{b}.weight", True)
            for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                m[f"{p}.mlp.shared.{a}.weight"] = (f"{h}.mlp.shared_expert.{b}.weight", True)
            m[f"{p}.mlp.shared_gate.weight"] = (f"{h}.mlp.shared_expert_gate.weight", True)
    m["norm.weight"] = ("model.norm.weight", False)
    m["head.weight"] = ("lm_head.weight", True)
    return m


def to_hf_tensors(model: Decoder, style: str = "llama") -> "OrderedDict[str, torch.Tensor]":
    """The model's weights under Hugging Face names and orientation."""
    spec = model.spec
    idr = idrak_tensors(model)
    m = hf_name_map(spec, style)
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    if style == "gpt2":
        for i in range(spec.layers):
            p, h = f"layers.{i}", f"transformer.h.{i}"
            out[f"{h}.attn.c_attn.weight"] = torch.cat([idr.pop(f"{p}.attn.{x}.weight") for x in "qkv"], dim=1)
            if f"{p}.attn.q.bias" in idr:
                out[f"{h}.attn.c_attn.bias"] = torch.cat([idr.pop(f"{p}.attn.{x}.bias") for x in "qkv"])
    for name, t in idr.items():
        if name not in m:
            raise KeyError(f"no Hugging Face name for '{name}' in style '{style}'")
        hf, tr = m[name]
        out[hf] = t.t().contiguous() if tr else t
    return out


def from_hf_tensors(spec: DecoderSpec, src: Mapping[str, torch.Tensor], style: str = "llama") -> Dict[str, torch.Tensor]:
    """Hugging Face tensors -> Idrak layout dict (ready for :func:`load_idrak_tensors`)."""
    m = hf_name_map(spec, style)
    out: Dict[str, torch.Tensor] = {}
    H, Hkv, D = spec.heads, spec.kv_heads, spec.head_dim
    if style == "gpt2":
        for i in range(spec.layers):
            p, h = f"layers.{i}", f"transformer.h.{i}"
            w = src[f"{h}.attn.c_attn.weight"]
            sizes = [H * D, Hkv * D, Hkv * D]
            for x, part in zip("qkv", torch.split(w, sizes, dim=1)):
                out[f"{p}.attn.{x}.weight"] = part.contiguous()
            if f"{h}.attn.c_attn.bias" in src:
                for x, part in zip("qkv", torch.split(src[f"{h}.attn.c_attn.bias"], sizes)):
                    out[f"{p}.attn.{x}.bias"] = part.contiguous()
    for name, (hf, tr) in m.items():
        if hf in src:
            out[name] = src[hf].t().contiguous() if tr else src[hf]
    if spec.tie_embeddings:
        out.pop("head.weight", None)
    elif "head.weight" not in out and "embed.weight" in out:
        out["head.weight"] = out["embed.weight"].t().contiguous()
    return out
