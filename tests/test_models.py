"""Decoder families against Hugging Face transformers and llama.cpp-converted GGUF fixtures (CPU, fp32)."""
import json
import os
import shutil
import warnings

import pytest
import torch

from idrak_b200.formats.gguf import GgufFile
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.models.families import architectures, spec_from_hf_config
from idrak_b200.models.pretrained import load_pretrained, save_huggingface, save_idrak

REF = os.path.join(os.environ.get("IDRAK_REFERENCE_DATA", ""), "gguf")
needs_ref = pytest.mark.skipif(not os.path.isdir(REF), reason="IDRAK_REFERENCE_DATA does not name the fixture folder")


@needs_ref
def test_gguf_dequantisers_are_bit_exact():
    with GgufFile(os.path.join(REF, "quants.gguf")) as f:
        assert f.metadata["test.string"] == "héllo" and f.metadata["test.numbers"] == [1, 2, 3]
        types = [n[2:] for n in f.tensors if n.startswith("q.")]
        assert len(types) == 14
        for t in types:
            assert torch.equal(f.read("q." + t).reshape(-1), f.read("expected." + t).reshape(-1)), t


@needs_ref
@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen3-q8", "tiny-gemma", "tiny-gemma2", "tiny-gemma3"])
def test_gguf_model_equals_huggingface_folder(name):
    hf = load_pretrained(os.path.join(REF, name + "-hf"))
    gg = load_pretrained(os.path.join(REF, name + ".gguf"))
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, hf.spec.vocabulary, (2, 24), generator=g)
    assert (hf(ids) - gg(ids)).abs().max().item() < 1e-5


@needs_ref
@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen3-q8", "tiny-gemma", "tiny-gemma2", "tiny-gemma3"])
def test_decoder_matches_transformers(name, tmp_path):
    transformers = pytest.importorskip("transformers")
    warnings.filterwarnings("ignore")
    src = os.path.join(REF, name + "-hf")
    folder = tmp_path / name
    shutil.copytree(src, folder)
    cfg = json.loads((folder / "config.json").read_text())
    if "model_type" not in cfg:
        cfg["model_type"] = {"LlamaForCausalLM": "llama", "Qwen3ForCausalLM": "qwen3"}[cfg["architectures"][0]]
        (folder / "config.json").write_text(json.dumps(cfg))
    mine = load_pretrained(folder)
    ref = transformers.AutoModelForCausalLM.from_pretrained(str(folder), dtype=torch.float32,
                                                            attn_implementation="eager").eval()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, mine.spec.vocabulary, (2, 20), generator=g)
    with torch.no_grad():
        assert (mine(ids) - ref(ids).logits).abs().max().item() < 2e-5


def test_gpt2_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    cfg = transformers.GPT2Config(vocab_size=300, n_positions=64, n_embd=64, n_layer=2, n_head=4,
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    ref = transformers.GPT2LMHeadModel(cfg).eval()
    ref.save_pretrained(tmp_path / "gpt2", safe_serialization=True)
    mine = load_pretrained(tmp_path / "gpt2")
    ids = torch.randint(0, 300, (2, 32))
    with torch.no_grad():
        assert (mine(ids) - ref(ids).logits).abs().max().item() < 2e-5
    # and back: our Hugging Face export loads into transformers with the same logits
    save_huggingface(mine, tmp_path / "out")
    again = transformers.GPT2LMHeadModel.from_pretrained(str(tmp_path / "out")).eval()
    with torch.no_grad():
        assert (again(ids).logits - ref(ids).logits).abs().max().item() < 2e-5


def test_llama_export_round_trips_through_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=200, max_positions=64,
                             theta=500000.0)
    m = build_decoder(spec, seed=5)
    save_huggingface(m, tmp_path / "hf")
    ref = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32,
                                                            attn_implementation="eager").eval()
    ids = torch.randint(0, 200, (2, 16))
    with torch.no_grad():
        assert (m(ids) - ref(ids).logits).abs().max().item() < 2e-5
    save_idrak(m, tmp_path / "idrak")
    m2 = load_pretrained(tmp_path / "idrak")
    assert torch.equal(m(ids), m2(ids))


def test_families_cover_the_reference_plugins_and_specs_round_trip():
    for a in ("LlamaForCausalLM", "MistralForCausalLM", "MixtralForCausalLM", "Qwen2ForCausalLM",
              "Qwen3ForCausalLM", "Qwen3MoeForCausalLM", "GemmaForCausalLM", "Gemma2ForCausalLM",
              "Gemma3ForCausalLM", "GPT2LMHeadModel"):
        assert a in architectures()
    spec, style = spec_from_hf_config({
        "architectures": ["Qwen2MoeForCausalLM"], "vocab_size": 100, "hidden_size": 32, "intermediate_size": 64,
        "num_hidden_layers": 4, "num_attention_heads": 4, "num_key_value_heads": 2, "num_experts": 4,
        "num_experts_per_tok": 2, "moe_intermediate_size": 16, "shared_expert_intermediate_size": 32,
        "decoder_sparse_step": 2, "mlp_only_layers": [3], "rope_scaling": {"rope_type": "yarn", "factor": 4.0,
                                                                           "original_max_position_embeddings": 32}})
    assert spec.experts == 4 and list(spec.expert_layers) == [False, True, False, False]
    assert spec.rope.scaling == "yarn" and spec.qkv_bias
    again = DecoderSpec.from_json(json.loads(spec.dumps()))
    assert again == spec
    m = build_decoder(spec, seed=0)
    assert sum(p.numel() for p in m.parameters()) >= spec.parameter_count
    ids = torch.randint(0, 100, (1, 8))
    assert m(ids).shape == (1, 8, 100) and torch.isfinite(m.loss(ids[:, :-1], ids[:, 1:]))
    with pytest.raises(ValueError, match="unknown keys"):
        DecoderSpec.from_json({"vocabulary": 1, "bogus": 2})


def test_tiny_gpt_trains_on_cpu():
    """Config 1 of the baseline: 4 layers, d_model 128, byte vocabulary, AdamW 3e-4, loss must fall."""
    from idrak_b200.ops import FusedAdamW
    spec = DecoderSpec.tiny_gpt()
    m = build_decoder(spec, seed=0)
    opt = FusedAdamW(m.decay_groups(0.1), lr=3e-3, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(1)
    data = torch.randint(0, 256, (8, 129), generator=g)
    first = last = None
    for step in range(12):
        opt.zero_grad()
        loss = m.loss(data[:, :-1], data[:, 1:])
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    assert abs(first - 5.545) < 0.2 and last < first - 0.5


def test_packed_spans_equal_separate_sequences_on_the_host():
    """``spans`` turn into one lower key bound per position; logits of a packed row equal those of each sequence run
    alone (host statement of what the attention kernels do in one launch)."""
    import torch
    from idrak_b200 import ops
    from idrak_b200.models import DecoderSpec, build_decoder
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=97, max_positions=64)
    model = build_decoder(spec, seed=3).float().eval()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 97, (1, 40), generator=g)
    spans = [(0, 13), (13, 14), (14, 40)]
    pos = torch.cat([torch.arange(hi - lo) for lo, hi in spans]).to(torch.int32)
    rs = ops.row_starts_from_spans(spans, 1, 40)
    assert rs[0, 12].item() == 0 and rs[0, 13].item() == 13 and rs[0, 39].item() == 14
    with torch.no_grad():
        packed = model(ids, pos, spans=spans)
        for lo, hi in spans:
            alone = model(ids[:, lo:hi], pos[lo:hi])
            assert torch.allclose(packed[:, lo:hi], alone, atol=1e-4, rtol=1e-4)


def test_expert_parameters_stay_views_of_the_stacked_buffers():
    """Moving or casting the module re-stacks; an optimizer step on the per-expert parameters changes the stacked
    arrays the grouped kernels read; loading a state dict writes through."""
    import torch
    from idrak_b200.models import DecoderSpec, build_decoder
    spec = DecoderSpec.llama(layers=1, dim=64, heads=2, kv_heads=2, ff_dim=128, vocab=50, max_positions=32)
    spec.experts, spec.experts_per_token, spec.expert_ff_dim = 4, 2, 64
    model = build_decoder(spec, seed=1)
    moe = model.blocks[0].mlp
    for m in (model, model.to(torch.bfloat16), model.float()):
        up, down = moe._stacked_now()
        assert up.shape == (4, 128, 64) and down.shape == (4, 64, 64)
        assert all(e.up_weight.data_ptr() == up[i].data_ptr() for i, e in enumerate(moe.experts))
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    ids = torch.randint(0, 50, (2, 16))
    model.loss(ids, ids).backward()
    before = moe._stacked[0].clone()
    opt.step()
    assert moe._stacked_now() is not None and not torch.equal(before, moe._stacked[0])
    sd = {k: torch.zeros_like(v) for k, v in model.state_dict().items()}
    model.load_state_dict(sd)
    assert moe._stacked_now() is not None and float(moe._stacked[0].abs().sum()) == 0.0
    moe.experts[1].up_weight.data = torch.ones(128, 64)          # re-homed by someone else: the loop path takes over
    assert moe._stacked_now() is None
