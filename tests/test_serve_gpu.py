"""Paged prefill / decode on the GPU against the training forward of the same bf16 model (teacher-forced), and an
end-to-end engine run with sampling on the device."""
import dataclasses

import pytest
import torch

from idrak_b200.models.decoder import build_decoder
from idrak_b200.models.spec import DecoderSpec
from idrak_b200.serve import GenerationOptions, LLMEngine
from idrak_b200.serve.runner import ModelRunner, PrefillItem

pytestmark = pytest.mark.gpu


def _spec(kind):
    if kind == "gpt2":
        return DecoderSpec.gpt2(layers=2, dim=256, heads=4, vocab=1000, max_positions=512)
    if kind == "llama128":
        return DecoderSpec.llama(layers=2, dim=256, heads=2, kv_heads=1, ff_dim=512, vocab=1000, max_positions=512)
    s = DecoderSpec.llama(layers=2, dim=256, heads=4, kv_heads=2, ff_dim=512, vocab=1000, max_positions=512)
    if kind == "windowed":
        s = dataclasses.replace(s, sliding_window=48)
    return s


@pytest.mark.parametrize("kind", ["llama", "llama128", "gpt2", "windowed"])
def test_paged_prefill_and_decode_match_forward(kind):
    dev = torch.device("cuda:0")
    spec = _spec(kind)
    model = build_decoder(spec, seed=5).to(dev, torch.bfloat16).eval()
    runner = ModelRunner(model, num_blocks=64, block_size=16)
    g = torch.Generator().manual_seed(1)
    lens = [37, 64, 5]
    steps = 70
    seqs = [torch.randint(0, spec.vocabulary, (n + steps,), generator=g).tolist() for n in lens]
    tables, nxt = [], 0
    for n in lens:
        need = (n + steps + 15) // 16
        tables.append(list(range(nxt, nxt + need)))
        nxt += need
    with torch.no_grad():
        full = [model(torch.tensor([s], dtype=torch.int32, device=dev))[0].float() for s in seqs]
    got = runner.prefill([PrefillItem(s[:n], 0, t) for s, n, t in zip(seqs, lens, tables)])
    for i, n in enumerate(lens):
        torch.testing.assert_close(got[i, : spec.vocabulary].float(), full[i][n - 1], rtol=3e-2, atol=3e-2)
    width = max(len(t) for t in tables)
    table = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device=dev)
    for k in range(steps):
        tok = torch.tensor([s[n + k] for s, n in zip(seqs, lens)], dtype=torch.int32, device=dev)
        pos = torch.tensor([n + k for n in lens], dtype=torch.int32, device=dev)
        lg = runner.decode(tok, pos, table)
        for i, n in enumerate(lens):
            torch.testing.assert_close(lg[i, : spec.vocabulary].float(), full[i][n + k], rtol=3e-2, atol=4e-2)
    # a shared prefix: the second half of a prompt computed against cached keys equals the whole prompt
    s, t = seqs[1], list(range(nxt, nxt + 5))
    runner.prefill([PrefillItem(s[:32], 0, t)])
    again = runner.prefill([PrefillItem(s[32:64], 32, t)])
    torch.testing.assert_close(again[0, : spec.vocabulary].float(), full[1][63], rtol=3e-2, atol=3e-2)


def test_engine_end_to_end_on_device():
    dev = torch.device("cuda:0")
    spec = _spec("llama")
    model = build_decoder(spec, seed=5).to(dev, torch.bfloat16).eval()
    for p in model.parameters():
        p.data.mul_(2.0)
    eng = LLMEngine(model, num_blocks=256, max_batch=16)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1000, (int(n),), generator=g).tolist() for n in torch.randint(4, 90, (24,), generator=g)]
    greedy = eng.generate(prompts, GenerationOptions.greedy_options(32))
    assert all(len(r.output) == 32 for r in greedy)
    # greedy tokens are the arg-max of the training forward wherever its top-2 margin is clear
    checked = 0
    for p, r in list(zip(prompts, greedy))[:6]:
        ids = p + r.output
        with torch.no_grad():
            lg = model(torch.tensor([ids], dtype=torch.int32, device=dev))[0].float()
        top = lg.topk(2, -1)
        for k, tok in enumerate(r.output):
            row = len(p) - 1 + k
            if float(top.values[row, 0] - top.values[row, 1]) > 0.25:
                assert int(top.indices[row, 0]) == tok
                checked += 1
    assert checked > 50
    o = GenerationOptions(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=3, max_tokens=24,
                          return_logprobs=True)
    a = eng.generate(prompts[:8], o)
    b = eng.generate(prompts[:8], o)
    assert [r.output for r in a] == [r.output for r in b]            # seeded sampling repeats
    assert all(len(r.logprobs) == 24 and max(r.logprobs) <= 0 for r in a)
    st = eng.stats()
    assert st["free_blocks"] == 256 and st["running"] == 0
