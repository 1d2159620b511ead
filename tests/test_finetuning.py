"""FineTuner on CPU: example encoding and loss masks, first-fit packing, a short LoRA run that lowers the loss and
writes a PEFT folder that loads back, DPO, non-finite step handling and resume."""
import json
import math
import os

import pytest
import torch

from idrak_b200.adapters.lora import add_adapters, adapter_parameters
from idrak_b200.adapters.peft import load_adapters
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.text import ByteTokenizer
from idrak_b200.text.finetuning import (IGNORE, FineTuner, FineTuningOptions, _lr_at, encode_example, pack_batches)


def _model(seed=1):
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=256)
    model = build_decoder(spec, seed=seed).float()
    model.head.data.mul_(20.0)       # the frozen head must be able to express confident predictions
    return model, tok


def test_encode_examples_and_masks():
    _, tok = _model()
    ids, train = encode_example({"prompt": "ab", "response": "cd"}, tok)
    assert ids == [97, 98, 99, 100, tok.eos_token_ids[0]] and train == [False, False, True, True, True]
    ids, train = encode_example({"text": "hey"}, tok)
    assert all(train) and ids[-1] == tok.eos_token_ids[0]
    msgs = {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
                         {"role": "user", "content": "more"}, {"role": "assistant", "content": "ok"}]}
    ids, train = encode_example(msgs, tok)
    text = tok.decode(ids)
    trained = tok.decode([i for i, t in zip(ids, train) if t])
    assert text.count("<|im_start|>") == 4 and trained == "yo<|im_end|>\nok<|im_end|>\n"
    with pytest.raises(ValueError):
        encode_example({"question": "?"}, tok)


def test_packing_first_fit_spans_and_targets():
    enc = [([1] * 10, [True] * 10), ([2] * 30, [False] * 15 + [True] * 15), ([3] * 25, [True] * 25), ([4] * 5, [True] * 5)]
    batches = pack_batches(enc, batch_tokens=64, max_length=40, packing=True)
    # rows: [10 + 30] and [25 + 5]; each row is 40 tokens, so two batches of one row... 64 holds only one 40-row
    assert len(batches) == 2
    b = batches[0]
    assert b.spans[:2] == [(0, 10), (10, 40)] and b.ids.shape[1] % 8 == 0
    assert b.positions[:10].tolist() == list(range(10)) and b.positions[10:40].tolist() == list(range(30))
    assert b.targets[0, 9].item() == IGNORE                      # the last token of a sequence predicts nothing
    assert (b.targets[0, 10:24] == IGNORE).all() and (b.targets[0, 24:39] == 2).all()
    assert b.trained_tokens == 9 + 15
    unpacked = pack_batches(enc, batch_tokens=64, max_length=40, packing=False)
    assert sum(len(x.spans) for x in unpacked) >= 4 and len(unpacked) == 2       # 10 + 30 | 25 + 5 tokens
    o = FineTuningOptions(learning_rate=1.0, warmup_fraction=0.1)
    assert _lr_at(0, 100, o) == pytest.approx(0.1) and _lr_at(9, 100, o) == pytest.approx(1.0)
    assert _lr_at(99, 100, o) < 0.01 and _lr_at(55, 100, o) == pytest.approx(0.5, abs=0.02)


def test_lora_run_lowers_loss_saves_and_resumes(tmp_path):
    model, tok = _model()
    data = [{"prompt": f"say {w}: ", "response": w * 3} for w in ("ab", "cd", "ef", "gh")] * 3
    o = FineTuningOptions(rank=4, alpha=8, learning_rate=3e-2, batch_tokens=128, max_length=64, epochs=20, base="bf16",
                          save_every=4, eval_every=4, warmup_fraction=0.1)
    seen = []
    res = FineTuner.train(model, tok, data, evaluation=data[:4], options=o, out_dir=str(tmp_path / "out"),
                          progress=lambda s, l: seen.append(s))
    assert res.steps == len(seen) > 6 and res.losses[-1] < 0.7 * res.losses[0]
    assert res.eval_losses and res.eval_losses[-1][1] < res.losses[0]
    assert all(not p.requires_grad for n, p in model.named_parameters() if "adapters" not in n)
    folder = tmp_path / "out"
    cfg = json.loads((folder / "adapter_config.json").read_text())
    assert cfg["r"] == 4 and cfg["peft_type"] == "LORA" and (folder / "adapter_model.safetensors").exists()
    fresh, _ = _model()
    add_adapters(fresh, 4, 8)
    load_adapters(fresh, str(folder))
    a = torch.cat([p.reshape(-1) for p in adapter_parameters(model)])
    b = torch.cat([p.reshape(-1) for p in adapter_parameters(fresh)])
    assert torch.allclose(a, b)
    # resume from the step-4 checkpoint reproduces the rest of the run (same seeded order)
    ck = folder / "checkpoint-4"
    assert (ck / "optimizer.safetensors").exists() and json.loads((ck / "train-state.json").read_text())["step"] == 4
    again, _ = _model()
    o2 = FineTuningOptions(**{**o.__dict__, "resume_from": str(ck), "save_every": 0, "eval_every": 0})
    res2 = FineTuner.train(again, tok, data, options=o2)
    assert res2.steps == res.steps and res2.losses[-1] == pytest.approx(res.losses[-1], rel=1e-4)


def test_dpo_prefers_chosen_and_non_finite_steps_stop():
    model, tok = _model()
    pairs = [{"prompt": "q: ", "chosen": "yes yes", "rejected": "no no"}] * 4
    o = FineTuningOptions(rank=4, alpha=8, learning_rate=5e-2, loss="dpo", dpo_beta=0.5, max_length=32, max_steps=12,
                          warmup_fraction=0.1)
    res = FineTuner.train(model, tok, pairs, options=o)
    assert res.losses[0] == pytest.approx(math.log(2), rel=1e-3)       # policy == reference at the start
    assert res.losses[-1] < 0.5 * res.losses[0]
    model2, _ = _model()
    ft = FineTuner(model2, tok, FineTuningOptions(rank=2, non_finite_steps=3, max_length=32))
    ft.batch_loss = lambda b: torch.tensor(float("nan"), requires_grad=True)
    with pytest.raises(FloatingPointError, match="3 steps in a row"):
        ft.fit([{"text": "abcdef"}] * 4)
    assert ft.result.skipped_steps == 3 and ft.result.steps == 0


def test_orpo_and_simpo_need_no_reference_and_prefer_the_chosen_answer():
    """Closed forms on hand-made mean log-probabilities, then a short run of each through the tuner."""
    from idrak_b200.text.finetuning import PREFERENCE_LOSSES, orpo_from_means, simpo_from_means
    a_c, a_r = torch.tensor(-0.5), torch.tensor(-1.5)
    odds = lambda a: a - math.log(1 - math.exp(a) + 1e-7)
    want = 0.5 - 0.1 * math.log(1 / (1 + math.exp(-(odds(-0.5) - odds(-1.5)))))
    assert float(orpo_from_means(a_c, a_r, 0.1)) == pytest.approx(want, rel=1e-5)
    assert float(simpo_from_means(a_c, a_r, 2.0, 1.0)) == pytest.approx(math.log(1 + math.exp(-(2.0 * 1.0 - 1.0))), rel=1e-5)
    assert float(simpo_from_means(a_r, a_c, 2.0, 1.0)) > float(simpo_from_means(a_c, a_r, 2.0, 1.0))
    assert {"dpo", "orpo", "simpo"} <= set(PREFERENCE_LOSSES)
    pairs = [{"prompt": "q: ", "chosen": "yes yes", "rejected": "no no"}] * 4
    for name in ("orpo", "simpo"):
        model, tok = _model()
        o = FineTuningOptions(rank=4, alpha=8, learning_rate=5e-2, loss=name, max_length=32, max_steps=12,
                              warmup_fraction=0.1)
        res = FineTuner.train(model, tok, pairs, options=o)
        assert res.losses[-1] < 0.7 * res.losses[0], (name, res.losses[0], res.losses[-1])
    model, tok = _model()
    with pytest.raises(ValueError, match="unknown loss"):
        FineTuner(model, tok, FineTuningOptions(loss="ppo", max_length=32)).batches(pairs)


def test_activation_estimate_and_ladder():
    from idrak_b200.models import DecoderSpec
    from idrak_b200.text import activation_memory as am
    spec = DecoderSpec.llama(layers=32, dim=4096, heads=32, kv_heads=8, ff_dim=14336, vocab=128256, max_positions=4096)
    held = am.estimate(spec, 8192, "held", adapter_rank=16)
    ckpt = am.estimate(spec, 8192, "checkpoint_blocks", adapter_rank=16)
    assert 25 < held.gib < 60                          # the measured LoRA step holds ~ 36 GiB above the weights at 8192 tokens
    assert ckpt.total_bytes < held.total_bytes / 6
    assert am.choose_policy(spec, 8192, 200 << 30).policy == "held"
    assert am.choose_policy(spec, 8192, 20 << 30).policy == "checkpoint_blocks"
    assert am.choose_policy(spec, 8192, 1 << 20).policy == "checkpoint_blocks"      # the last rung even when nothing fits
    assert am.next_rung("held") == "checkpoint_blocks" and am.next_rung("checkpoint_blocks") is None


def test_fine_tuner_steps_down_the_ladder_on_out_of_memory(monkeypatch):
    torch.manual_seed(0)
    tok = _tokenizer() if "_tokenizer" in globals() else None
    if tok is None:
        from idrak_b200.text import ByteTokenizer
        tok = ByteTokenizer()
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.text.finetuning import FineTuner, FineTuningOptions
    model = build_decoder(DecoderSpec.llama(layers=2, dim=32, heads=2, kv_heads=2, ff_dim=64, vocab=tok.vocab_size, max_positions=128), seed=0)
    ft = FineTuner(model, tok, FineTuningOptions(rank=4, alpha=8.0, max_steps=3, batch_tokens=64, max_length=64))
    calls = {"n": 0}
    real = ft.batch_loss

    def flaky(b):
        calls["n"] += 1
        if calls["n"] == 1:
            raise torch.OutOfMemoryError("simulated")
        return real(b)
    monkeypatch.setattr(ft, "batch_loss", flaky)
    res = ft.fit([{"prompt": "hello ", "completion": "world " * 3} for _ in range(6)])
    assert res.steps == 3 and res.activation_policy == "checkpoint_blocks" and model.checkpoint_blocks is True
    monkeypatch.setattr(ft, "batch_loss", lambda b: (_ for _ in ()).throw(torch.OutOfMemoryError("again")))
    ft.o.max_steps = 5
    import pytest as _pytest
    with _pytest.raises(torch.OutOfMemoryError):
        ft.fit([{"prompt": "hello ", "completion": "world"}])


def test_flat_data_parallel_ranks_start_and_stay_equal(tmp_path):
    """Two gloo ranks that drew different random numbers before building the tuner: the adapters are a function of the
    options' seed (and are broadcast), so one gradient all-reduce per step keeps the ranks bit-identical."""
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    out = tmp_path / "flat.pt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29931", os.path.join(here, "finetune_flat_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    got = torch.load(out)
    assert got["start"] and got["end"]
    assert len(got["losses"]) == 4 and got["losses"][-1] < got["losses"][0]
