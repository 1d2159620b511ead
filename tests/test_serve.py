"""Continuous-batching engine on CPU: scheduler behaviour, and token-exact agreement of paged generation with
the plain forward pass (greedy), under prefix sharing and under block pressure that forces preemption."""
import pytest
import torch

from idrak_b200.models.decoder import build_decoder
from idrak_b200.models.spec import DecoderSpec
from idrak_b200.serve import GenerationOptions, LLMEngine, QueueFull, Scheduler
from idrak_b200.serve.scheduler import DECODE, PREFILL


def _model(kind="llama", **kw):
    if kind == "llama":
        import dataclasses
        spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=200, max_positions=128)
        spec = dataclasses.replace(spec, **kw)
    else:
        spec = DecoderSpec.gpt2(layers=2, dim=64, heads=4, vocab=200, max_positions=128)
    m = build_decoder(spec, seed=1).float().eval()
    for p in m.parameters():
        p.data.mul_(3.0)          # sharper logits: arg-max is stable against summation order
    return m


def _naive(model, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        with torch.no_grad():
            lg = model(torch.tensor([ids], dtype=torch.int32))
        ids.append(int(lg[0, -1].argmax()))
    return ids[len(prompt):]


def test_scheduler_admission_queue_limit_and_deadline():
    s = Scheduler(num_blocks=8, block_size=16, max_batch=2, max_prefill_tokens=64, queue_limit=3, prefix_sharing=False)
    s.add(1, list(range(20)), 4)
    s.add(2, list(range(20)), 4)
    s.add(3, list(range(5)), 4, deadline=1.0)
    with pytest.raises(QueueFull):
        s.add(4, [1, 2], 2)
    with pytest.raises(ValueError):
        Scheduler(2, 16, 2, 64, 0, False).add(9, list(range(40)), 10)
    kind, ids, expired = s.step(0.0)
    assert kind == PREFILL and ids == [1, 2] and expired == []
    assert s.commit(1, 7, False) is False and s.commit(2, 7, False) is False
    kind, ids, expired = s.step(2.0)           # the batch is full; request 3 timed out waiting
    assert kind == DECODE and ids == [1, 2] and expired == [3]
    assert s.commit(1, 7, True) is True
    st = s.stats()
    assert st["running"] == 1 and st["rejected"] == 1 and st["free_blocks"] == 6


def test_scheduler_shares_prompt_prefix_blocks():
    s = Scheduler(8, 16, 4, 256, 0, True)
    prompt = list(range(40))
    s.add(1, prompt, 2)
    assert s.step(0.0)[1] == [1]
    s.commit(1, 5, False)
    s.add(2, prompt[:33] + [99, 98], 2)
    assert s.step(0.0)[1] == [2]
    a, b = s.info(1), s.info(2)
    assert b.cached_prefix == 32 and s.blocks(1, 8)[:2] == s.blocks(2, 8)[:2]
    assert s.blocks(1, 8)[2] != s.blocks(2, 8)[2] and a.cached_prefix == 0


@pytest.mark.parametrize("kind", ["llama", "gpt2"])
def test_engine_matches_plain_forward(kind):
    m = _model(kind)
    eng = LLMEngine(m, num_blocks=12, block_size=16, max_batch=4, prefix_sharing=True)
    prompts = [[5, 6, 7, 8, 9] * 4 + [i] for i in range(6)] + [[3, 4]]
    outs = eng.generate(prompts, GenerationOptions.greedy_options(20))
    for p, r in zip(prompts, outs):
        assert r.output == _naive(m, p, 20) and r.finish_reason == "length"
    st = eng.stats()
    assert st["prefix_hits"] > 0 and st["free_blocks"] == 12


def test_engine_preempts_and_recomputes_under_block_pressure():
    m = _model()
    eng = LLMEngine(m, num_blocks=6, block_size=16, max_batch=4, prefix_sharing=False)
    prompts = [[10 + i, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23] for i in range(4)]
    outs = eng.generate(prompts, GenerationOptions.greedy_options(30))
    assert eng.stats()["preemptions"] > 0
    for p, r in zip(prompts, outs):
        assert r.output == _naive(m, p, 30)


def test_engine_windowed_and_softcapped_attention_paths():
    m = _model(sliding_window=8)
    eng = LLMEngine(m, num_blocks=12, max_batch=2)
    p = list(range(30, 50))
    assert eng.generate([p], GenerationOptions.greedy_options(12))[0].output == _naive(m, p, 12)
    m = _model(attention_softcap=20.0, logit_softcap=30.0)
    eng = LLMEngine(m, num_blocks=12, max_batch=2)
    outs = eng.generate([p, p[:17]], GenerationOptions.greedy_options(12))
    assert outs[0].output == _naive(m, p, 12) and outs[1].output == _naive(m, p[:17], 12)


def test_engine_stop_tokens_sampling_and_late_arrivals():
    m = _model()
    eng = LLMEngine(m, num_blocks=16, max_batch=4, eos_token_ids=[])
    ref = _naive(m, [1, 2, 3], 10)
    r = eng.generate([[1, 2, 3]], GenerationOptions.greedy_options(10, stop_token_ids=(ref[4],)))[0]
    stop_at = ref.index(ref[4])
    assert r.finish_reason == "stop" and r.output == ref[: stop_at + 1]
    # sampled requests with one seed repeat exactly; a request added mid-flight joins the running batch
    o = GenerationOptions(temperature=0.9, top_k=20, top_p=0.95, seed=7, max_tokens=12, return_logprobs=True)
    a = eng.add_request([4, 5, 6], o)
    for _ in range(3):
        eng.step()
    b = eng.add_request([9, 9, 9], GenerationOptions.greedy_options(5))
    while not (eng.requests[a].finished and eng.requests[b].finished):
        eng.step()
    ra, rb = eng.release(a), eng.release(b)
    assert len(ra.output) == 12 and len(ra.logprobs) == 12 and all(lp <= 0 for lp in ra.logprobs)
    assert rb.output == _naive(m, [9, 9, 9], 5)
    with pytest.raises(ValueError):
        eng.add_request(list(range(128)))


def test_engine_abort_and_queue_timeout():
    m = _model()
    t = [0.0]
    eng = LLMEngine(m, num_blocks=16, max_batch=1, clock=lambda: t[0])
    seen = []
    a = eng.add_request([1, 2, 3], GenerationOptions.greedy_options(50))
    b = eng.add_request([4, 5, 6], GenerationOptions.greedy_options(5, timeout=1.0), on_token=seen.append)
    eng.step()
    t[0] = 5.0
    eng.step()
    assert eng.requests[b].finish_reason == "timeout" and seen[-1].finished and seen[-1].token == -1
    eng.abort(a)
    assert eng.requests[a].finish_reason == "abort" and not eng.has_work()
    assert eng.stats()["free_blocks"] == 16


def test_engine_with_an_int8_kv_cache_generates_like_the_bf16_cache():
    """The same greedy continuation (CPU path) with the cache held as int8 codes + scales: first tokens equal, the
    cache tensors really are int8, and block accounting counts the scales."""
    import torch
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.serve import GenerationOptions, LLMEngine
    from idrak_b200.serve.runner import ModelRunner
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=300, max_positions=128)
    model = build_decoder(spec, seed=3).eval()
    prompts = [list(range(5, 25)), list(range(40, 47))]
    opts = GenerationOptions.greedy_options(6)
    a = LLMEngine(model, num_blocks=32, max_batch=4, prefix_sharing=False, use_graph=False)
    b = LLMEngine(model, num_blocks=32, max_batch=4, prefix_sharing=False, use_graph=False, kv_dtype=torch.int8)
    out_a = [r.output for r in a.generate(prompts, opts)]
    out_b = [r.output for r in b.generate(prompts, opts)]
    assert b.runner.k_cache[0].dtype == torch.int8 and b.runner.k_scale[0] is not None
    assert [o[0] for o in out_a] == [o[0] for o in out_b]
    assert sum(x == y for oa, ob in zip(out_a, out_b) for x, y in zip(oa, ob)) >= 10
    assert ModelRunner.blocks_that_fit(spec, 1 << 20, 16, 1) > ModelRunner.blocks_that_fit(spec, 1 << 20, 16, 2)


def test_folding_the_norm_weights_into_the_projections_keeps_the_function():
    """``norm(x) W^T == (x rstd) (W diag(w))^T``: after the rewrite the norms have unit weight and logits are unchanged,
    through the training forward and through the engine."""
    import torch
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.serve import GenerationOptions, LLMEngine
    from idrak_b200.serve.runner import fold_norms_into_projections
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=97, max_positions=64)
    spec.tie_embeddings = False
    model = build_decoder(spec, seed=4).float().eval()
    with torch.no_grad():
        for blk in model.blocks:
            blk.attn_norm.weight.uniform_(0.5, 1.5)
            blk.mlp_norm.weight.uniform_(0.5, 1.5)
        model.norm.weight.uniform_(0.5, 1.5)
    ids = torch.randint(0, 97, (2, 20))
    with torch.no_grad():
        before = model(ids)
    want = LLMEngine(model, num_blocks=32, max_batch=2).generate([[5, 6, 7]], GenerationOptions.greedy_options(6))[0].output
    assert fold_norms_into_projections(model) and model._norms_folded
    assert float((model.blocks[0].attn_norm.weight.detach() - 1).abs().max()) == 0.0
    with torch.no_grad():
        after = model(ids)
    assert torch.allclose(before, after, atol=1e-4, rtol=1e-4)
    got = LLMEngine(model, num_blocks=32, max_batch=2, fold_norms=True).generate([[5, 6, 7]], GenerationOptions.greedy_options(6))[0].output
    assert got == want
    tied = build_decoder(DecoderSpec.gpt2(layers=1, dim=32, heads=2, vocab=50, max_positions=16), seed=1)
    assert not fold_norms_into_projections(tied)              # LayerNorm and a tied head: left alone
