import pytest
import torch

from idrak_b200.training.offload import GroupedOptimizer, HostOptimizer, LayerOffloader


def test_host_optimizer_follows_adamw_and_resumes():
    torch.manual_seed(0)
    a, b = torch.nn.Linear(6, 5), torch.nn.Linear(6, 5)
    b.load_state_dict(a.state_dict())
    ref = torch.optim.AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = HostOptimizer(b.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    x = torch.randn(16, 6)
    for _ in range(5):
        for m, o in ((a, ref), (b, opt)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-6)
    state = opt.state_dict()
    assert {"step", "m.0", "v.0", "master.1"} <= set(state) and int(state["step"]) == 5
    c = torch.nn.Linear(6, 5)
    again = HostOptimizer(c.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    again.load_state_dict(state)
    for m, o in ((b, opt), (c, again)):
        o.zero_grad()
        m(x).pow(2).mean().backward()
        o.step()
    for p, q in zip(b.parameters(), c.parameters()):
        assert torch.equal(p, q)
    # clipping and skipped non-finite steps
    clip = HostOptimizer(c.parameters(), lr=1e-2, max_grad_norm=1e-3)
    c.zero_grad()
    (c(x).sum() * 1e3).backward()
    before = [p.detach().clone() for p in c.parameters()]
    assert clip.step() > 1.0
    assert max((p - q).abs().max().item() for p, q in zip(c.parameters(), before)) < 2e-2
    c.weight.grad.fill_(float("nan"))
    kept = [p.detach().clone() for p in c.parameters()]
    clip.step()
    assert all(torch.equal(p, q) for p, q in zip(c.parameters(), kept)) and clip.step_count == 1


def test_grouped_optimizer():
    m = torch.nn.Sequential(torch.nn.Linear(3, 3), torch.nn.Linear(3, 1))
    g = GroupedOptimizer({"body": HostOptimizer(m[0].parameters(), lr=0.1), "head": torch.optim.SGD(m[1].parameters(), lr=0.5)})
    before = [p.detach().clone() for p in m.parameters()]
    m(torch.randn(4, 3)).sum().backward()
    g.step()
    assert all(not torch.equal(p, q) for p, q in zip(m.parameters(), before))
    g.zero_grad()
    assert all(p.grad is None for p in m.parameters())
    state = g.state_dict()
    assert set(state) == {"body", "head"}
    g.load_state_dict(state)
    with pytest.raises(KeyError, match="no group 'head'"):
        g.load_state_dict({"body": state["body"]})
    with pytest.raises(ValueError, match="more than one group"):
        GroupedOptimizer({"a": torch.optim.SGD(m.parameters(), lr=0.1), "b": torch.optim.SGD(m[1].parameters(), lr=0.1)})


def test_layer_offloader_on_cpu_keeps_results():
    torch.manual_seed(1)
    blocks = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh()) for _ in range(5)])
    x = torch.randn(3, 8)
    def run():
        h = x
        for b in blocks:
            h = b(h)
        return h
    ref = run()
    off = LayerOffloader(blocks, device="cpu", resident=2)
    assert torch.equal(run(), ref) and off.fetches == 3 * 1 + 0        # blocks 2..4 fetched once each (prefetch covers the next)
    assert torch.equal(run(), ref)
    off.remove()
    assert torch.equal(run(), ref)


@pytest.mark.gpu
def test_layer_offloader_streams_blocks_through_the_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.manual_seed(2)
    blocks = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(256, 256), torch.nn.GELU()) for _ in range(6)])
    x = torch.randn(32, 256)
    h = x
    with torch.no_grad():
        for b in blocks:
            h = b(h)
    off = LayerOffloader(blocks, device="cuda", resident=1)
    for _ in range(2):
        g = x.cuda()
        with torch.no_grad():
            for b in blocks:
                g = b(g)
        assert torch.allclose(g.cpu(), h, atol=1e-4)
    on_gpu = [next(b.parameters()).is_cuda for b in blocks]
    assert on_gpu == [True] + [False] * 5
    off.remove()
    assert all(next(b.parameters()).is_cuda for b in blocks)
    m = torch.nn.Linear(64, 64).cuda().bfloat16()
    opt = HostOptimizer(m.parameters(), lr=1e-2)
    w0 = m.weight.detach().clone()
    m(torch.randn(8, 64, device="cuda", dtype=torch.bfloat16)).float().pow(2).mean().backward()
    assert opt.step() > 0 and not torch.equal(m.weight, w0) and opt.master[0].is_pinned()
