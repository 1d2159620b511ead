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


@pytest.mark.parametrize("H,Hkv,Dh,rot", [(8, 2, 64, 64), (32, 8, 128, 128), (4, 4, 128, 64), (6, 2, 256, 128)])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_fused_norm_rope_kv_write_matches_the_separate_steps(H, Hkv, Dh, rot, qk_norm):
    """One launch = query / key RMS norm + RoPE (in place on the packed projection) + paged cache write; compared with
    the same steps composed on the CPU path of the op."""
    T, bs, nb = 45, 16, 12
    qkv = _rand((T, (H + 2 * Hkv) * Dh), 1)
    pos = torch.randint(0, 3000, (T,), dtype=torch.int32, device="cuda")
    slots = torch.randperm(nb * bs)[:T].to(torch.int32).cuda()
    slots[7] = -1
    qn = (_rand((Dh,), 2).float() * 0.1 + 1).to(torch.bfloat16) if qk_norm else None
    kn = (_rand((Dh,), 3).float() * 0.1 + 1).to(torch.bfloat16) if qk_norm else None
    kc = torch.zeros((nb, bs, Hkv, Dh), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    got = qkv.clone()
    D.norm_rope_kv(got, H, Hkv, Dh, pos, slots, kc, vc, None, None, qn, kn, 1e-6, 10000.0, rot)
    want = qkv.cpu().clone()
    kc2, vc2 = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    D.norm_rope_kv(want, H, Hkv, Dh, pos.cpu(), slots.cpu(), kc2, vc2, None, None,
                   qn.cpu() if qn is not None else None, kn.cpu() if kn is not None else None, 1e-6, 10000.0, rot)
    assert (got.float().cpu() - want.float()).abs().max().item() < 3e-2
    assert (kc.float().cpu() - kc2.float()).abs().max().item() < 3e-2
    assert torch.equal(vc.cpu(), vc2)                       # values are copied, bit for bit
    # what the cache holds for keys is exactly what stayed in the projection buffer
    k_rows = got[:, H * Dh:(H + Hkv) * Dh].unflatten(-1, (Hkv, Dh))
    keep = slots >= 0
    assert torch.equal(kc.view(-1, Hkv, Dh)[slots[keep].long()], k_rows[keep])


@pytest.mark.parametrize("H,Hkv,Dh", [(32, 8, 128), (12, 12, 64), (4, 1, 128)])
@pytest.mark.parametrize("splits", [1, 4, None])
def test_int8_kv_cache_write_and_decode(H, Hkv, Dh, splits):
    """int8 codes + one scale per (slot, kv head): the fused write against the plain quantiser, and decode attention
    over the codes against the reference over the de-quantised cache."""
    bs, nblocks, seqs, T = 16, 120, 4, 600
    lens = [1, 50, 333, 216]
    table = torch.randperm(nblocks)[: seqs * 24].reshape(seqs, 24).to(torch.int32).cuda()
    kc = torch.zeros((nblocks, bs, Hkv, Dh), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    ks = torch.zeros((nblocks, bs, Hkv), dtype=torch.float32, device="cuda")
    vs = torch.zeros_like(ks)
    qkv = _rand((T, (H + 2 * Hkv) * Dh), 5)
    slots, t = [], 0
    for s_, n in enumerate(lens):
        for p_ in range(n):
            slots.append(int(table[s_, p_ // bs]) * bs + p_ % bs)
    slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    D.norm_rope_kv(qkv, H, Hkv, Dh, None, slots, kc, vc, ks, vs)
    k_src = qkv[:, H * Dh:(H + Hkv) * Dh].unflatten(-1, (Hkv, Dh))
    q8, sc = D.quantize_kv_reference(k_src)
    got_codes = kc.view(-1, Hkv, Dh)[slots.long()].to(torch.int16)
    assert (got_codes - q8.to(torch.int16)).abs().max().item() <= 1          # division vs reciprocal at a tie
    assert torch.allclose(ks.view(-1, Hkv)[slots.long()], sc, rtol=1e-6)
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    q = _rand((seqs, H, Dh), 6)
    out = D.paged_decode(q, kc, vc, table, lens_t, splits=splits, k_scale=ks, v_scale=vs)
    ref = D.paged_decode_reference(q, kc, vc, table, lens_t, k_scale=ks, v_scale=vs)
    assert (out.float() - ref.float()).abs().max().item() < 2e-2
    # and close to attention over the unquantised keys / values (what the int8 cache costs)
    kb = torch.zeros((nblocks, bs, Hkv, Dh), dtype=torch.bfloat16, device="cuda")
    vb = torch.zeros_like(kb)
    D.norm_rope_kv(qkv, H, Hkv, Dh, None, slots, kb, vb)
    exact = D.paged_decode_reference(q, kb, vb, table, lens_t)
    assert (out.float() - exact.float()).abs().max().item() < 6e-2
