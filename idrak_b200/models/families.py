"""Model families: Hugging Face ``config.json`` -> ``DecoderSpec`` (and back), by architecture name.

Registered: Llama (2/3), Mistral, Mixtral, Qwen2, Qwen2-MoE, Qwen3, Qwen3-MoE, Gemma 1/2/3 (text), GPT-2.
A family is a function from the config dict to a spec plus the checkpoint naming style; apps can
``register`` their own, which shadows a built-in of the same architecture name.

Reference: PretrainedArchitectures / Architectures (src/Idrak/Models/Abstractions/PretrainedArchitectures.cs,
src/Idrak/Models/Architectures.cs) and the family plug-ins under src/Idrak.Text.Plugins/{Llama,Mistral,Qwen,Gemma}.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, Tuple

from .spec import DecoderSpec, RopeSettings

Family = Callable[[dict], Tuple[DecoderSpec, str]]
_REGISTRY: Dict[str, Family] = {}


def register(architecture: str, family: Family) -> None:
    _REGISTRY[architecture] = family


def architectures() -> list[str]:
    return sorted(_REGISTRY)


def _rope(cfg: dict, head_dim: int) -> RopeSettings:
    r = RopeSettings(theta=float(cfg.get("rope_theta", 10000.0)))
    prf = cfg.get("partial_rotary_factor")
    if prf and prf != 1.0:
        r.rotary_dim = int(head_dim * prf)
    sc = cfg.get("rope_scaling")
    if isinstance(sc, dict):
        kind = sc.get("rope_type", sc.get("type"))
        if kind in ("linear", "dynamic", "llama3", "yarn"):
            r.scaling = kind
            r.factor = float(sc.get("factor", 1.0))
            r.original_max_positions = sc.get("original_max_position_embeddings")
            r.low_freq_factor = float(sc.get("low_freq_factor", 1.0))
            r.high_freq_factor = float(sc.get("high_freq_factor", 4.0))
            r.beta_fast = float(sc.get("beta_fast", 32.0))
            r.beta_slow = float(sc.get("beta_slow", 1.0))
            r.attention_factor = sc.get("attention_factor")
        elif kind not in (None, "default"):
            raise NotImplementedError(f"rope_scaling type '{kind}' is not supported")
    return r


def _llama_like(cfg: dict, **over) -> DecoderSpec:
    dim, heads = int(cfg["hidden_size"]), int(cfg["num_attention_heads"])
    head_dim = int(cfg.get("head_dim") or dim // heads)
    kw = dict(
        vocabulary=int(cfg["vocab_size"]), dim=dim, layers=int(cfg["num_hidden_layers"]), heads=heads,
        kv_heads=int(cfg.get("num_key_value_heads") or heads), head_dim=head_dim,
        ff_dim=int(cfg["intermediate_size"]), max_positions=int(cfg.get("max_position_embeddings", 2048)),
        norm="rms", norm_epsilon=float(cfg.get("rms_norm_eps", 1e-6)), gated=True,
        activation={"silu": "silu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu", "relu": "relu"}.get(
            cfg.get("hidden_act", cfg.get("hidden_activation", "silu")), "silu"),
        rope=_rope(cfg, head_dim), qkv_bias=bool(cfg.get("attention_bias", False)),
        tie_embeddings=bool(cfg.get("tie_word_embeddings", False)))
    kw.update(over)
    return DecoderSpec(**kw)


def _llama(cfg):
    return _llama_like(cfg, feed_forward_bias=bool(cfg.get("mlp_bias", False))), "llama"


def _mistral(cfg):
    spec = _llama_like(cfg)
    if cfg.get("sliding_window"):
        spec.sliding_window = int(cfg["sliding_window"])
    return spec, "llama"


def _mixtral(cfg):
    spec, style = _mistral(cfg)
    spec.experts = int(cfg.get("num_local_experts", 0))
    spec.experts_per_token = int(cfg.get("num_experts_per_tok", 2))
    return spec, style


def _qwen2(cfg):
    spec = _llama_like(cfg, qkv_bias=True)
    if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
        spec.sliding_window = int(cfg["sliding_window"])
        first = int(cfg.get("max_window_layers", 0))
        spec.sliding_window_layers = [i >= first for i in range(spec.layers)]
    return spec, "llama"


def _qwen3(cfg):
    spec = _llama_like(cfg, qk_norm=True)
    return spec, "llama"


def _qwen_moe(base):
    def fam(cfg):
        spec, style = base(cfg)
        spec.experts = int(cfg.get("num_experts", 0))
        spec.experts_per_token = int(cfg.get("num_experts_per_tok", 0))
        spec.expert_ff_dim = int(cfg.get("moe_intermediate_size", 0))
        spec.shared_expert_ff_dim = int(cfg.get("shared_expert_intermediate_size", 0) or 0)
        spec.normalize_top_k = bool(cfg.get("norm_topk_prob", False))
        step = int(cfg.get("decoder_sparse_step", 1) or 1)
        only = set(cfg.get("mlp_only_layers") or [])
        spec.expert_layers = [((i + 1) % step == 0) and i not in only for i in range(spec.layers)]
        return spec, style
    return fam


def _gemma(version: int):
    def fam(cfg):
        if "text_config" in cfg:
            cfg = {**cfg["text_config"], "tie_word_embeddings": cfg.get("tie_word_embeddings", True)}
        spec = _llama_like(cfg, norm_offset=1.0, tie_embeddings=True, activation="gelu")
        spec.embedding_scale = float(spec.dim) ** 0.5
        if version >= 2:
            spec.post_norms = True
            q = cfg.get("query_pre_attn_scalar")
            if q:
                spec.attention_scale = float(q) ** -0.5
            spec.attention_softcap = cfg.get("attn_logit_softcapping")
            spec.logit_softcap = cfg.get("final_logit_softcapping")
            if cfg.get("sliding_window"):
                spec.sliding_window = int(cfg["sliding_window"])
                types = cfg.get("layer_types")
                if types:
                    spec.sliding_window_layers = [t == "sliding_attention" for t in types]
                elif version == 2:
                    spec.sliding_window_layers = [i % 2 == 0 for i in range(spec.layers)]
                else:
                    pat = int(cfg.get("sliding_window_pattern", 6))
                    spec.sliding_window_layers = [(i + 1) % pat != 0 for i in range(spec.layers)]
        if version >= 3:
            spec.qk_norm = True
            local = cfg.get("rope_local_base_freq")
            if local:
                spec.sliding_window_rope = RopeSettings(theta=float(local))
        return spec, "llama"
    return fam


def _gpt2(cfg):
    spec = DecoderSpec.gpt2(layers=int(cfg["n_layer"]), dim=int(cfg["n_embd"]), heads=int(cfg["n_head"]),
                            vocab=int(cfg["vocab_size"]), max_positions=int(cfg.get("n_positions", 1024)),
                            ff_dim=cfg.get("n_inner") or None, dropout=0.0)
    spec.norm_epsilon = float(cfg.get("layer_norm_epsilon", 1e-5))
    return spec, "gpt2"


for _name, _fam in {
    "LlamaForCausalLM": _llama, "MistralForCausalLM": _mistral, "MixtralForCausalLM": _mixtral,
    "Qwen2ForCausalLM": _qwen2, "Qwen2MoeForCausalLM": _qwen_moe(_qwen2), "Qwen3ForCausalLM": _qwen3,
    "Qwen3MoeForCausalLM": _qwen_moe(_qwen3), "GemmaForCausalLM": _gemma(1), "Gemma2ForCausalLM": _gemma(2),
    "Gemma3ForCausalLM": _gemma(3), "Gemma3ForConditionalGeneration": _gemma(3), "GPT2LMHeadModel": _gpt2,
}.items():
    register(_name, _fam)


def spec_from_hf_config(cfg: dict | str | Path) -> Tuple[DecoderSpec, str]:
    """(spec, checkpoint naming style) for a Hugging Face configuration (dict, JSON text or path)."""
    if isinstance(cfg, (str, Path)):
        p = Path(cfg)
        cfg = json.loads(p.read_text() if p.exists() else str(cfg))
    archs = cfg.get("architectures") or []
    for a in archs:
        if a in _REGISTRY:
            return _REGISTRY[a](cfg)
    mt = cfg.get("model_type")
    by_type = {"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "mixtral": "MixtralForCausalLM",
               "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "gemma": "GemmaForCausalLM",
               "gemma2": "Gemma2ForCausalLM", "gemma3_text": "Gemma3ForCausalLM", "gpt2": "GPT2LMHeadModel",
               "qwen2_moe": "Qwen2MoeForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM"}
    if mt in by_type:
        return _REGISTRY[by_type[mt]](cfg)
    raise NotImplementedError(f"no family registered for architectures {archs} / model_type {mt}; "
                              f"registered: {architectures()}")


def hf_config_from_spec(spec: DecoderSpec, style: str = "llama") -> dict:
    """A Hugging Face configuration that describes ``spec`` (what ``save_huggingface`` writes)."""
    if style == "gpt2":
        return {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "vocab_size": spec.vocabulary,
                "n_embd": spec.dim, "n_layer": spec.layers, "n_head": spec.heads, "n_positions": spec.max_positions,
                "n_inner": spec.ff_dim, "layer_norm_epsilon": spec.norm_epsilon,
                "activation_function": "gelu_new", "tie_word_embeddings": True}
    cfg = {"architectures": ["Qwen3ForCausalLM" if spec.qk_norm else "LlamaForCausalLM"],
           "model_type": "qwen3" if spec.qk_norm else "llama", "vocab_size": spec.vocabulary,
           "hidden_size": spec.dim, "intermediate_size": spec.ff_dim, "num_hidden_layers": spec.layers,
           "num_attention_heads": spec.heads, "num_key_value_heads": spec.kv_heads, "head_dim": spec.head_dim,
           "max_position_embeddings": spec.max_positions, "rms_norm_eps": spec.norm_epsilon,
           "rope_theta": spec.rope.theta if spec.rope else 10000.0, "tie_word_embeddings": spec.tie_embeddings,
           "hidden_act": "silu" if spec.activation == "silu" else "gelu_pytorch_tanh",
           "attention_bias": spec.qkv_bias, "torch_dtype": "float32"}
    if spec.rope and spec.rope.scaling:
        cfg["rope_scaling"] = {"rope_type": spec.rope.scaling, "factor": spec.rope.factor,
                               "original_max_position_embeddings": spec.rope.original_max_positions}
    return cfg
