import math

import pytest
import torch

from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.rag import Bm25Index, Chunk, Hit, reciprocal_rank_fusion, rerank
from idrak_b200.text import distillation as D
from idrak_b200.text import evaluation as E


def _model(vocab=64, dim=32, seed=0):
    return build_decoder(DecoderSpec.llama(layers=2, dim=dim, heads=2, kv_heads=2, ff_dim=64, vocab=vocab, max_positions=128), seed=seed)


def test_perplexity_scores_every_token_once():
    m = _model().eval()
    toks = torch.randint(0, 64, (150,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = E.perplexity(m, toks, window=150, stride=150)
    with torch.no_grad():
        lp = torch.log_softmax(m(torch.tensor([toks])).float(), -1)[0, :-1, :64]
    nll = -lp.gather(-1, torch.tensor(toks[1:])[:, None]).mean().item()
    assert whole.tokens == 149 and abs(whole.nll - nll) < 1e-4 and abs(whole.perplexity - math.exp(nll)) < 1e-2
    strided = E.perplexity(m, toks, window=64, stride=32, batch=3)
    assert strided.tokens == 149 and abs(strided.nll - whole.nll) < 0.2       # shorter contexts, same tokens
    assert abs(strided.bits_per_token - strided.nll / math.log(2)) < 1e-9
    with pytest.raises(ValueError):
        E.perplexity(m, [1])


def test_answer_scoring():
    m = _model().eval()
    prompt, cands = [5, 6, 7], [[1, 2], [3], [4, 8, 9]]
    s = E.score_continuations(m, prompt, cands)
    with torch.no_grad():
        for c, got in zip(cands, s):
            lp = torch.log_softmax(m(torch.tensor([prompt + c])).float(), -1)[0]
            want = sum(lp[len(prompt) - 1 + j, t].item() for j, t in enumerate(c))
            assert abs(got - want) < 1e-4
    n = E.score_continuations(m, prompt, cands, normalise=True)
    assert abs(n[2] - s[2] / 3) < 1e-6
    best = max(range(3), key=n.__getitem__)
    assert E.multiple_choice_accuracy(m, [{"prompt": prompt, "choices": cands, "answer": best}]) == 1.0
    assert E.exact_match("The Eiffel Tower!", ["eiffel tower"]) == 1.0 and E.exact_match("tower", ["eiffel tower"]) == 0.0
    assert abs(E.token_f1("the tall eiffel tower", ["eiffel tower"]) - 0.8) < 1e-9 and E.token_f1("x", ["y"]) == 0.0


def test_topk_cache_and_distillation_loss(tmp_path):
    torch.manual_seed(0)
    s_logits, t_logits = torch.randn(2, 5, 40), torch.randn(2, 5, 40) * 2
    full = D.TeacherTopK.from_logits(t_logits, k=40, temperature=2.0)
    # with every token kept the loss is the cross-entropy H(teacher, student) * T^2
    lt = torch.log_softmax(t_logits / 2, -1)
    ls = torch.log_softmax(s_logits / 2, -1)
    want = -(lt.exp() * ls).sum(-1).mean() * 4
    assert abs(D.topk_distillation_loss(s_logits, full, 2.0).item() - want.item()) < 5e-3
    part = D.TeacherTopK.from_logits(t_logits, k=8)
    assert part.indices.shape == (2, 5, 8) and (part.rest.float().exp() < 0.9).all()
    mask = torch.tensor([[1, 1, 0, 0, 0], [1, 0, 0, 0, 0]])
    assert D.topk_distillation_loss(s_logits, part, 1.0, mask).item() > 0
    part.save(str(tmp_path / "t.safetensors"))
    again = D.TeacherTopK.load(str(tmp_path / "t.safetensors"))
    assert torch.equal(again.indices, part.indices) and torch.equal(again.values, part.values)


def test_distiller_pulls_the_student_towards_the_teacher():
    teacher = _model(seed=1)
    with torch.no_grad():
        teacher.head.mul_(8)                                       # a teacher with opinions
    ids = torch.randint(0, 64, (8, 24), generator=torch.Generator().manual_seed(3))
    for kw in ({}, {"top_k": 16}):
        student = _model(dim=16, seed=2)
        opt = torch.optim.AdamW(student.parameters(), lr=5e-3)
        d = D.Distiller(student, teacher, opt, alpha=0.2, temperature=1.5, **kw)
        first = d.step(ids)
        for _ in range(25):
            last = d.step(ids)
        assert last["teacher_loss"] < first["teacher_loss"] and "grad_norm" in last
    with torch.no_grad():
        cached = D.TeacherTopK.from_logits(teacher(ids[:, :-1]).float()[..., :64], 16, 1.5)
    d = D.Distiller(student, None, opt, alpha=0.0, temperature=1.5)
    assert d.step(ids, cached=cached)["teacher_loss"] > 0


def test_bm25_fusion_and_rerank():
    docs = ["the cat sat on the mat", "dogs chase cats in the park", "quantum computers use qubits",
            "a cat and a dog became friends", "parks are full of dogs and people walking"]
    idx = Bm25Index([Chunk(t, f"d{i}") for i, t in enumerate(docs)])
    hits = idx.search("cat", k=3)
    assert [h.index for h in hits][:2] == [0, 3] and all(h.score > 0 for h in hits) and len(hits) == 2   # "cats" is another word
    assert idx.search("qubits quantum")[0].index == 2 and idx.search("zebra") == []
    # rare words weigh more than common ones
    assert idx.search("the qubits")[0].index == 2
    a = [Hit(idx.chunks[i], 1.0, i) for i in (0, 1, 2)]
    b = [Hit(idx.chunks[i], 1.0, i) for i in (3, 1, 0)]
    fused = reciprocal_rank_fusion([a, b], k=3)
    assert [h.index for h in fused] == [0, 1, 3] or [h.index for h in fused][0] in (0, 1)
    assert abs(fused[0].score - (1 / 61 + 1 / 63)) < 1e-12 or abs(fused[0].score - 2 / 62) < 1e-12
    rr = rerank("q", a, score=lambda pairs: [len(p[1]) for p in pairs], k=2)
    assert [h.index for h in rr] == [2, 1] and rerank("q", [], score=lambda p: []) == []
