"""Fused softmax cross-entropy, chunked token loss and fused AdamW/SGD vs PyTorch."""
import pytest
import torch

from idrak_b200 import ops

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,vocab,ld", [(64, 1000, 1000), (33, 50257, 50304), (8, 128256, 128256), (16, 257, 264)])
def test_softmax_xent_loss_and_grad(rows, vocab, ld):
    logits = _rand((rows, ld), 2.0, 1)
    g = torch.Generator(device="cuda").manual_seed(2)
    t = torch.randint(0, vocab, (rows,), generator=g, device="cuda")
    t[0] = -100
    ref_l = logits[:, :vocab].float().requires_grad_()
    loss_ref = torch.nn.functional.cross_entropy(ref_l, t, ignore_index=-100, reduction="none")
    loss_ref.sum().backward()
    work = logits.clone()
    losses = ops.softmax_xent_(work, t, vocab, 1.0, -100, True)
    assert (losses - loss_ref).abs().max().item() < 2e-2
    assert (work[:, :vocab].float() - ref_l.grad).abs().max().item() < 1e-2
    assert work[:, vocab:].abs().max().item() == 0 if ld > vocab else True


@pytest.mark.parametrize("rows,vocab,ld", [(300, 1000, 1000), (301, 50257, 50304), (1024, 257, 264), (777, 32000, 32000)])
def test_softmax_xent_pipelined_rows(rows, vocab, ld):
    """Enough rows for one persistent CTA per SM with two rows in flight (the bulk-copy kernel): loss, gradient,
    zero padding columns, an ignored row, the no-gradient mode leaving the logits untouched, and equal bits on a
    second run."""
    logits = _rand((rows, ld), 2.0, 5)
    g = torch.Generator(device="cuda").manual_seed(6)
    t = torch.randint(0, vocab, (rows,), generator=g, device="cuda")
    t[3] = -100
    t[5] = vocab - 1
    ref_l = logits[:, :vocab].float().requires_grad_()
    loss_ref = torch.nn.functional.cross_entropy(ref_l, t, ignore_index=-100, reduction="none")
    loss_ref.sum().backward()
    keep = logits.clone()
    only = ops.softmax_xent_(keep, t, vocab, 1.0, -100, False)
    assert torch.equal(keep, logits)
    assert (only - loss_ref).abs().max().item() < 2e-2
    work = logits.clone()
    losses = ops.softmax_xent_(work, t, vocab, 0.5, -100, True)
    assert (losses - loss_ref).abs().max().item() < 2e-2
    assert (work[:, :vocab].float() - 0.5 * ref_l.grad).abs().max().item() < 1e-2
    assert work[3].abs().max().item() == 0
    if ld > vocab:
        assert work[:, vocab:].abs().max().item() == 0
    again = logits.clone()
    losses2 = ops.softmax_xent_(again, t, vocab, 0.5, -100, True)
    assert torch.equal(again, work) and torch.equal(losses, losses2)


def test_token_cross_entropy_chunked_matches_torch():
    T, C, V, Vp = 512, 256, 1000, 1024
    h = _rand((T, C), 1.0, 1).requires_grad_()
    w = _rand((Vp, C), 0.05, 2).requires_grad_()
    g = torch.Generator(device="cuda").manual_seed(3)
    t = torch.randint(0, V, (T,), generator=g, device="cuda")
    loss = ops.token_cross_entropy(h, w, t, vocab=V, chunk_rows=200, ignore_index=None)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = torch.nn.functional.cross_entropy((hr @ wr.t())[:, :V], t)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    assert (h.grad.float() - hr.grad).abs().max().item() < 2e-2 * hr.grad.abs().max().item() + 1e-5
    assert (w.grad.float() - wr.grad).abs().max().item() < 3e-2 * wr.grad.abs().max().item() + 1e-5


def test_fused_adamw_matches_torch_adamw():
    torch.manual_seed(0)
    shapes = [(300, 77), (5000,), (64, 64), (3,)]
    ps = [torch.randn(s, device="cuda").to(torch.bfloat16).requires_grad_() for s in shapes]
    ref = [p.detach().float().clone().requires_grad_() for p in ps]
    opt = ops.FusedAdamW([{"params": ps[:2], "weight_decay": 0.1}, {"params": ps[2:], "weight_decay": 0.0}],
                         lr=1e-2, betas=(0.9, 0.95), eps=1e-8, max_grad_norm=1.0)
    ropt = torch.optim.AdamW([{"params": ref[:2], "weight_decay": 0.1}, {"params": ref[2:], "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in range(3):
        for p, r in zip(ps, ref):
            g = torch.randn_like(r)
            p.grad = g.to(torch.bfloat16)
            r.grad = p.grad.float()
        norm_ref = torch.nn.utils.clip_grad_norm_(ref, 1.0)
        opt.step()
        ropt.step()
        assert abs(opt.grad_norm() - norm_ref.item()) < 1e-2 * norm_ref.item()
        for m, r in zip(opt.master, ref):
            assert (m - r).abs().max().item() < 1e-5
    for p, m in zip(ps, opt.master):
        assert torch.equal(p, m.to(torch.bfloat16))


def test_fused_sgd_momentum():
    torch.manual_seed(1)
    p = torch.randn(1000, device="cuda").to(torch.bfloat16).requires_grad_()
    r = p.detach().float().clone().requires_grad_()
    opt = ops.FusedSGD([p], lr=0.1, momentum=0.9)
    ropt = torch.optim.SGD([r], lr=0.1, momentum=0.9)
    for _ in range(3):
        g = torch.randn(1000, device="cuda")
        p.grad, r.grad = g.to(torch.bfloat16), g.to(torch.bfloat16).float()
        opt.step(); ropt.step()
    assert (opt.master[0] - r).abs().max().item() < 1e-5
