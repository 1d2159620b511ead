"""Speculative decoding reproduces the target's greedy output; beam search of width 1 is greedy search and wider
beams never score worse. CPU."""
import pytest
import torch

from idrak_b200.generation.beam import BeamSearch
from idrak_b200.generation.speculative import SpeculativeDecoder
from idrak_b200.models import DecoderSpec, build_decoder


def _model(seed, layers=2, dim=64):
    spec = DecoderSpec.llama(layers=layers, dim=dim, heads=4, kv_heads=2, ff_dim=2 * dim, vocab=120, max_positions=256)
    m = build_decoder(spec, seed=seed).float().eval()
    for p in m.parameters():
        p.data.mul_(3.0)
    return m


def _greedy(model, prompt, n):
    ids = list(prompt)
    lps = 0.0
    for _ in range(n):
        with torch.no_grad():
            lg = model(torch.tensor([ids], dtype=torch.int32))[0, -1].float()
        lp = torch.log_softmax(lg, -1)
        t = int(lp.argmax())
        lps += float(lp[t])
        ids.append(t)
    return ids[len(prompt):], lps


@pytest.mark.parametrize("lookahead", [1, 3, 5])
def test_speculative_greedy_equals_target_greedy(lookahead):
    target, draft = _model(1), _model(2, layers=1)
    prompt = [5, 9, 11, 3, 7, 2]
    want, _ = _greedy(target, prompt, 24)
    res = SpeculativeDecoder(target, draft, max_tokens=128, lookahead=lookahead).generate(prompt, 24)
    assert res.tokens == want and res.target_passes <= 24 and res.proposed >= res.accepted >= 0
    # the target as its own draft: everything is accepted, k + 1 tokens per pass
    same = SpeculativeDecoder(target, target, max_tokens=128, lookahead=lookahead).generate(prompt, 24)
    assert same.tokens == want and same.acceptance == 1.0 and same.target_passes <= -(-24 // (lookahead + 1)) + 1
    stop = SpeculativeDecoder(target, draft, max_tokens=128, lookahead=lookahead).generate(prompt, 24, eos_token_ids=[want[5]])
    assert stop.tokens == want[: want.index(want[5]) + 1]


def test_speculative_sampling_runs_and_repeats_with_its_seed():
    target, draft = _model(1), _model(2, layers=1)
    d = SpeculativeDecoder(target, draft, max_tokens=128, lookahead=3)
    a = d.generate([1, 2, 3], 16, temperature=0.9, seed=4).tokens
    b = SpeculativeDecoder(target, draft, max_tokens=128, lookahead=3).generate([1, 2, 3], 16, temperature=0.9, seed=4).tokens
    assert len(a) == 16 and a == b


def test_beam_search_width_one_is_greedy_and_wider_is_no_worse():
    m = _model(3)
    prompt = [4, 8, 15, 16, 23, 42]
    want, lp = _greedy(m, prompt, 12)
    one = BeamSearch(m, width=1, max_tokens=64).search(prompt, 12)[0]
    assert one.tokens == want and one.logprob == pytest.approx(lp, rel=1e-4, abs=1e-4)
    wide = BeamSearch(m, width=4, max_tokens=64, early_stopping=False).search(prompt, 12, n_best=3)
    assert len(wide) == 3 and wide[0].score >= one.score - 1e-5 and wide[0].score >= wide[1].score >= wide[2].score
    # the best hypothesis's log-probability is what the model assigns to it
    ids = prompt + wide[0].tokens
    with torch.no_grad():
        lg = torch.log_softmax(m(torch.tensor([ids], dtype=torch.int32))[0].float(), -1)
    check = sum(float(lg[len(prompt) - 1 + i, t]) for i, t in enumerate(wide[0].tokens))
    assert wide[0].logprob == pytest.approx(check, rel=1e-3, abs=1e-3)
    eos = want[3]
    hyp = BeamSearch(m, width=3, max_tokens=64).search(prompt, 12, eos_token_ids=[eos], n_best=3)
    assert any(h.finished and h.tokens[-1] == eos for h in hyp)
