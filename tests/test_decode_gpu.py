"""Paged decode attention, paged KV writes and the device sampler vs plain PyTorch."""
import pytest
import torch

from idrak_b200.ops import decode as D

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)


@pytest.mark.parametrize("H,Hkv,Dh", [(4, 1, 128), (32, 8, 128), (12, 12, 64), (8, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3, None])
def test_paged_decode_matches_reference(H, Hkv, Dh, splits):
    bs, nblocks, seqs = 16, 200, 5
    k_cache, v_cache = _rand((nblocks, bs, Hkv, Dh), 1), _rand((nblocks, bs, Hkv, Dh), 2)
    lens = torch.tensor([1, 17, 333, 64, 500], dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(nblocks, generator=g)[: seqs * 32].reshape(seqs, 32).to(torch.int32).cuda()
    q = _rand((seqs, H, Dh), 4)
    out = D.paged_decode(q, k_cache, v_cache, table, lens, splits=splits)
    ref = D.paged_decode_reference(q, k_cache, v_cache, table, lens)
    assert (out.float() - ref.float()).abs().max().item() < 2e-2
    outw = D.paged_decode(q, k_cache, v_cache, table, lens, window=100, splits=splits)
    refw = D.paged_decode_reference(q, k_cache, v_cache, table, lens, window=100)
    assert (outw.float() - refw.float()).abs().max().item() < 2e-2


def test_kv_write_paged_from_fused_qkv():
    H, Hkv, Dh, T, bs = 8, 2, 64, 37, 16
    qkv = _rand((T, (H + 2 * Hkv) * Dh), 1)
    k = qkv[:, H * Dh:(H + Hkv) * Dh].unflatten(-1, (Hkv, Dh))
    v = qkv[:, (H + Hkv) * Dh:].unflatten(-1, (Hkv, Dh))
    kc = torch.zeros((10, bs, Hkv, Dh), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    slots = (torch.randperm(160)[:T]).to(torch.int32).cuda()
    slots[5] = -1
    D.kv_write_paged(k, v, slots, kc, vc)
    flat_k, flat_v = kc.view(-1, Hkv, Dh), vc.view(-1, Hkv, Dh)
    for t in range(T):
        if t == 5:
            continue
        assert torch.equal(flat_k[slots[t]], k[t]) and torch.equal(flat_v[slots[t]], v[t])
    assert int((flat_k.abs().sum((1, 2)) > 0).sum()) == T - 1


def test_argmax_and_sampler():
    rows, V, ld = 7, 50257, 50304
    logits = _rand((rows, ld), 1) * 3
    ids = D.argmax_rows(logits, V)
    assert torch.equal(ids.cpu(), logits[:, :V].float().argmax(-1).to(torch.int32).cpu())
    dev = "cuda"
    t = torch.full((rows,), 0.8, device=dev)
    seeds = torch.arange(rows, dtype=torch.int64, device=dev) + 11
    # top_k = 1 is greedy whatever the seed
    one = D.sample_rows(logits, V, t, torch.ones(rows, dtype=torch.int32, device=dev), torch.ones(rows, device=dev),
                        torch.zeros(rows, device=dev), seeds, 0)
    assert torch.equal(one, ids)
    k = torch.full((rows,), 40, dtype=torch.int32, device=dev)
    p = torch.full((rows,), 0.9, device=dev)
    a = D.sample_rows(logits, V, t, k, p, torch.zeros(rows, device=dev), seeds, 3)
    b = D.sample_rows(logits, V, t, k, p, torch.zeros(rows, device=dev), seeds, 3)
    c = D.sample_rows(logits, V, t, k, p, torch.zeros(rows, device=dev), seeds, 4)
    assert torch.equal(a, b)                       # same (seed, step) -> same draw
    top40 = torch.topk(logits[:, :V].float(), 40, dim=-1).indices
    for r in range(rows):
        assert int(a[r]) in top40[r].tolist() and int(c[r]) in top40[r].tolist()
    # empirical frequencies follow the filtered distribution
    row = logits[:1].repeat(4000, 1).contiguous()
    n = row.shape[0]
    draws = D.sample_rows(row, V, torch.ones(n, device=dev), torch.full((n,), 4, dtype=torch.int32, device=dev),
                          torch.ones(n, device=dev), torch.zeros(n, device=dev),
                          torch.arange(n, dtype=torch.int64, device=dev), 0)
    vals, idx = torch.topk(logits[0, :V].float(), 4)
    want = torch.softmax(vals, 0)
    got = torch.stack([(draws == i).float().mean() for i in idx])
    assert (got - want).abs().max().item() < 0.04
    # a heavy repetition penalty moves the choice away from a token in the history
    hist = ids.reshape(rows, 1).contiguous()
    pen = D.sample_rows(logits, V, t, torch.ones(rows, dtype=torch.int32, device=dev), torch.ones(rows, device=dev),
                        torch.zeros(rows, device=dev), seeds, 0, history=hist,
                        repeat_penalty=torch.full((rows,), 50.0, device=dev))
    assert not torch.equal(pen, ids)


def test_sampler_ties_do_not_crowd_out_larger_logits():
    """All-equal logits with a few larger ones (a masked vocabulary looks like this): the larger ones must all be
    candidates, the tied places go to the lowest ids, and the draw repeats."""
    rows, V = 4, 4096
    dev = "cuda"
    logits = torch.zeros(rows, V, device=dev, dtype=torch.float32)
    big = [4000, 4010, 4095]
    for j, b in enumerate(big):
        logits[:, b] = 5.0 + j
    t = torch.ones(rows, device=dev)
    ones, zeros = torch.ones(rows, device=dev), torch.zeros(rows, device=dev)
    seeds = torch.arange(rows, dtype=torch.int64, device=dev)
    greedy = D.sample_rows(logits, V, t, torch.ones(rows, dtype=torch.int32, device=dev), ones, zeros, seeds, 0)
    assert greedy.tolist() == [4095] * rows
    k = torch.full((rows,), 8, dtype=torch.int32, device=dev)
    allowed = set(big) | {0, 1, 2, 3, 4}              # three larger logits, then five ties by ascending id
    seen = set()
    for step in range(200):
        a = D.sample_rows(logits, V, t, k, ones, zeros, seeds, step)
        b = D.sample_rows(logits, V, t, k, ones, zeros, seeds, step)
        assert torch.equal(a, b)
        seen |= set(a.tolist())
    assert seen <= allowed and set(big) <= seen, sorted(seen)
