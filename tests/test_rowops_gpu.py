"""Row-wise kernels (norms, activations, RoPE, embedding, column sums) vs plain PyTorch fp32."""
import pytest
import torch

from idrak_b200 import ops

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * (b.abs().max().item() + 1e-3), f"err {err}"


@pytest.mark.parametrize("rows,C", [(7, 64), (300, 768), (129, 1024), (33, 4096), (5, 8192)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_forward_backward(rows, C, rms):
    x = _rand((rows, C), 1.0, 1).requires_grad_()
    w = (_rand((C,), 0.2, 2).float() + 1).to(torch.bfloat16).requires_grad_()
    b = None if rms else _rand((C,), 0.2, 3).requires_grad_()
    y = ops.rms_norm(x, w, 1e-5) if rms else ops.layer_norm(x, w, b, 1e-5)
    dy = _rand((rows, C), 1.0, 4)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    br = None if rms else b.detach().float().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        yr = torch.nn.functional.layer_norm(xr, (C,), wr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, 3e-2)
    if not rms:
        _close(b.grad, br.grad, 3e-2)


@pytest.mark.parametrize("rows,C", [(64, 64), (1000, 768), (4099, 1024), (16384, 768), (70, 256), (40, 4096)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_branch_adds_the_residual_gradient_and_leaves_column_sums(rows, C, rms):
    """``(norm(x), x)``: one backward kernel gives d(norm) + d(residual), the norm's parameter gradients and - where
    the row length fits the pipelined kernel - the column sums of that dx, which a following bias gradient reuses."""
    x = _rand((rows, C), 1.0, 1).requires_grad_()
    w = (_rand((C,), 0.2, 2).float() + 1).to(torch.bfloat16).requires_grad_()
    b = None if rms else _rand((C,), 0.2, 3).requires_grad_()
    y, xr_out = ops.norm_branch(x, w, b, 1e-5, rms)
    dy, dres = _rand((rows, C), 1.0, 4), _rand((rows, C), 1.0, 5)
    got = {}
    x.register_hook(lambda g: got.setdefault("dx", g))
    torch.autograd.backward([y, xr_out], [dy, dres])
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    br = None if rms else b.detach().float().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        yr = torch.nn.functional.layer_norm(xr, (C,), wr, br, 1e-5)
    torch.autograd.backward([yr, xr], [dy.float(), dres.float()])
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, 3e-2)
    if not rms:
        _close(b.grad, br.grad, 3e-2)
    tagged = getattr(got["dx"], "_idrak_colsum", None)
    from idrak_b200 import _native
    if _native.lib().idrak_norm_bwd_sums_dx(rows, C):
        assert 256 <= C <= 1024
        assert tagged is not None and tagged[1] == got["dx"]._version
        want = got["dx"].float().sum(0)
        assert (tagged[0] - want).abs().max().item() <= 1e-3 * max(1.0, want.abs().max().item())
        # deterministic: a second pass gives the same bits
        x2 = x.detach().clone().requires_grad_()
        y2, r2 = ops.norm_branch(x2, w.detach().requires_grad_(), None if rms else b.detach().requires_grad_(), 1e-5, rms)
        again = {}
        x2.register_hook(lambda g: again.setdefault("dx", g))
        torch.autograd.backward([y2, r2], [dy, dres])
        assert torch.equal(again["dx"], got["dx"]) and torch.equal(again["dx"]._idrak_colsum[0], tagged[0])


def test_bias_gradient_reuses_the_sums_left_by_the_norm_backward():
    """linear (with bias) -> pre-norm block input: the bias gradient must equal the one computed by a column-sum pass,
    and an in-place change of the gradient tensor must make the stale sums unusable."""
    from idrak_b200.ops.gemm import bias_grad
    dy = _rand((512, 768), 1.0, 7)
    ref = ops.colsum(dy)
    dy._idrak_colsum = (dy.float().sum(0), dy._version)
    got = bias_grad(dy.reshape(-1, 768), None, dy)
    _close(got, ref, 1e-2)
    dy.add_(1.0)                                    # version moves on: the attached sums no longer describe dy
    got = bias_grad(dy.reshape(-1, 768), None, dy)
    _close(got, dy.float().sum(0), 1e-2)


def test_norm_with_residual_sum():
    x, r = _rand((64, 768), 1.0, 1), _rand((64, 768), 1.0, 2)
    w, b = _rand((768,), 1.0, 3), _rand((768,), 1.0, 4)
    out, mean, rstd, summed = ops.norm_forward(x, w, b, 1e-5, False, residual=r)
    s_ref = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(summed, s_ref)
    _close(out, torch.nn.functional.layer_norm(s_ref.float(), (768,), w.float(), b.float(), 1e-5))


def test_gelu_and_gated():
    x = _rand((128, 3072), 2.0, 1).requires_grad_()
    y = ops.gelu(x)
    dy = _rand(x.shape, 1.0, 2)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(xr, approximate="tanh")
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    for kind in ("silu", "gelu", "relu", "tanh"):
        gu = _rand((96, 2 * 1024), 1.5, 3).requires_grad_()
        o = ops.gated_activation(gu, kind)
        do = _rand(o.shape, 1.0, 4)
        o.backward(do)
        gr = gu.detach().float().requires_grad_()
        from idrak_b200.ops.rowops import _gate_ref, GATE_KINDS
        orf = _gate_ref(gr[:, :1024], GATE_KINDS[kind]) * gr[:, 1024:]
        orf.backward(do.float())
        _close(o, orf)
        _close(gu.grad, gr.grad)


def test_rope_matches_reference_and_inverts():
    x = _rand((50, 8, 64), 1.0, 1)
    pos = torch.arange(50, device="cuda", dtype=torch.int32) + 3
    y = x.clone()
    ops.rope_(y, pos, 10000.0)
    _close(y, ops.rope_reference(x, pos, 10000.0))
    ops.rope_(y, pos, 10000.0, inverse=True)
    _close(y, x)


def test_embedding_forward_backward():
    V, C, B, S = 1000, 256, 4, 64
    wte, wpe = _rand((V, C), 1.0, 1).requires_grad_(), _rand((S, C), 1.0, 2).requires_grad_()
    g = torch.Generator(device="cuda").manual_seed(3)
    ids = torch.randint(0, 50, (B, S), generator=g, device="cuda")   # many repeats
    out = ops.embedding(ids, wte, wpe)
    do = _rand(out.shape, 1.0, 4)
    out.backward(do)
    wr, pr = wte.detach().float().requires_grad_(), wpe.detach().float().requires_grad_()
    outr = wr[ids] + pr[None, :S]
    outr.backward(do.float())
    _close(out, outr)
    _close(wte.grad, wr.grad)
    _close(wpe.grad, pr.grad)


def test_colsum():
    x = _rand((1000, 200), 1.0, 1)
    _close(ops.colsum(x), x.float().sum(0), 1e-2)
