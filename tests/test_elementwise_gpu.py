"""Element-wise, softmax / axis-sum / layout, CTC, recurrent-cell and convolution kernels against plain PyTorch fp32."""
import pytest
import torch

from idrak_b200.ops import conv as cv
from idrak_b200.ops import ctc as ctc_ops
from idrak_b200.ops import pointwise as pw
from idrak_b200.ops import recurrent as rc
from idrak_b200.ops import reduce as rd

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


def _input(name, n, dtype, g):
    x = torch.randn(n, generator=g, device=DEV)
    if name in ("sqrt", "log", "inv_sqrt", "pow", "reciprocal"):
        x = x.abs() + 0.5
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(pw.UNARY))
def test_unary_forward_backward(name, dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    n = 8 * 1000 + 5                                   # a vector body and a scalar tail
    a, b = {"affine": (1.5, -0.25), "pow": (2.5, 0), "clamp": (-0.5, 0.7), "leaky_relu": (0.1, 0),
            "inv_sqrt": (1e-3, 0)}.get(name, (0.0, 0.0))
    x = _input(name, n, dtype, g).requires_grad_(True)
    y = pw.unary(name, x, a, b)
    xr = x.detach().float().requires_grad_(True)
    yr = pw.unary_reference(name, xr, a, b)
    torch.testing.assert_close(y.float(), yr.to(dtype).float(), **_tol(dtype))
    dy = torch.randn(n, generator=g, device=DEV).to(dtype)
    y.backward(dy)
    yr.backward(dy.float())
    torch.testing.assert_close(x.grad.float(), xr.grad.to(dtype).float(), **_tol(dtype))
    acc = torch.ones_like(x.detach())
    pw.unary_backward(name, x.detach(), dy, a, b, accumulate_into=acc)
    torch.testing.assert_close(acc.float(), (1 + xr.grad).to(dtype).float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(pw.BINARY))
def test_binary_forward_backward(name, dtype):
    g = torch.Generator(device=DEV).manual_seed(4)
    n = 4099
    x = torch.randn(n, generator=g, device=DEV).to(dtype).requires_grad_(True)
    y0 = torch.randn(n, generator=g, device=DEV)
    if name == "div":
        y0 = y0.abs() + 0.5
    y = y0.to(dtype).requires_grad_(True)
    out = pw.binary(name, x, y, 0.5, -2.0)
    xr, yr = x.detach().float().requires_grad_(True), y.detach().float().requires_grad_(True)
    ref = pw.binary_reference(name, xr, yr, 0.5, -2.0)
    torch.testing.assert_close(out.float(), ref.to(dtype).float(), **_tol(dtype))
    dy = torch.randn(n, generator=g, device=DEV).to(dtype)
    out.backward(dy)
    ref.backward(dy.float())
    tol = dict(rtol=5e-2, atol=5e-2) if dtype == torch.bfloat16 else _tol(dtype)
    # on a tie max / min send the whole gradient to the first operand (PyTorch splits it): compare away from ties
    apart = (x.detach() != y.detach()) if name in ("max", "min") else torch.ones_like(x, dtype=torch.bool)
    torch.testing.assert_close(x.grad.float()[apart], xr.grad[apart], **tol)
    torch.testing.assert_close(y.grad.float()[apart], yr.grad[apart], **tol)
    if name in ("max", "min"):
        assert torch.equal(x.grad[~apart], dy[~apart]) and (y.grad[~apart] == 0).all()


def test_muladd_where_fill_rowvec():
    g = torch.Generator(device=DEV).manual_seed(5)
    x, y, z = (torch.randn(33, 40, generator=g, device=DEV, requires_grad=True) for _ in range(3))
    out = pw.muladd(x, y, z)
    torch.testing.assert_close(out, x * y + z)
    out.sum().backward()
    torch.testing.assert_close(x.grad, y.detach())
    cond = torch.rand(33, 40, generator=g, device=DEV) > 0.5
    a, b = x.detach().clone().requires_grad_(True), y.detach().clone().requires_grad_(True)
    w = pw.where(cond, a, b)
    assert torch.equal(w, torch.where(cond, a, b))
    w.sum().backward()
    assert torch.equal(a.grad, cond.float()) and torch.equal(b.grad, (~cond).float())
    t = torch.empty(1001, device=DEV, dtype=torch.bfloat16)
    assert (pw.fill_(t, 2.5) == 2.5).all()
    v = torch.randn(40, generator=g, device=DEV, requires_grad=True)
    xa = x.detach().clone().requires_grad_(True)
    r = pw.add_rowvec(xa, v)
    torch.testing.assert_close(r, xa + v)
    r.backward(torch.ones_like(r))
    torch.testing.assert_close(v.grad, torch.full((40,), 33.0, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_draws_the_same_mask_again(dtype):
    n, p, seed = 4096 + 3, 0.25, 1234567
    x = torch.ones(n, device=DEV, dtype=dtype, requires_grad=True)
    res = torch.full((n,), 2.0, device=DEV, dtype=dtype)
    y = pw.dropout(x, p, seed, residual=res)
    ref = pw.dropout_reference(x.detach().cpu(), p, seed, res.cpu())
    torch.testing.assert_close(y.detach().cpu().float(), ref.float(), **_tol(dtype))
    kept = (y.detach().float() - 2.0) > 0
    assert abs(kept.float().mean().item() - (1 - p)) < 0.03
    y.backward(torch.ones_like(y))
    assert torch.equal(x.grad.float() > 0, kept)                   # the backward pass drew the same mask
    assert torch.equal(pw.dropout(x, p, seed, residual=res), y)    # and so does a rerun
    assert pw.dropout(x, p, seed, training=False) is x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [7, 256, 1000, 5000])
@pytest.mark.parametrize("log", [False, True])
def test_softmax_rows(cols, dtype, log):
    g = torch.Generator(device=DEV).manual_seed(6)
    x = (3 * torch.randn(37, cols, generator=g, device=DEV)).to(dtype).requires_grad_(True)
    y = rd.softmax(x, log=log)
    xr = x.detach().float().requires_grad_(True)
    yr = torch.log_softmax(xr, -1) if log else torch.softmax(xr, -1)
    torch.testing.assert_close(y.float(), yr.to(dtype).float(), **_tol(dtype))
    dy = torch.randn(37, cols, generator=g, device=DEV).to(dtype)
    y.backward(dy)
    # the kernel differentiates the value it stored (rounded to the storage type)
    ys = y.detach().float()
    want = (dy.float() - ys.exp() * dy.float().sum(-1, keepdim=True)) if log else \
        ys * (dy.float() - (dy.float() * ys).sum(-1, keepdim=True))
    torch.testing.assert_close(x.grad.float(), want.to(dtype).float(), **_tol(dtype))


def test_scale_mask_softmax_matches_reference():
    g = torch.Generator(device=DEV).manual_seed(7)
    B, H, Tq, Tk = 2, 3, 20, 28
    s = torch.randn(B, H, Tq, Tk, generator=g, device=DEV)
    mask = torch.zeros(Tq, Tk, device=DEV)
    mask[:, :3] = float("-inf")
    got = rd.scale_mask_softmax(s, 0.3, mask, causal=True)
    want = rd.softmax_reference(s, 0.3, mask, True)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    # a row with nothing visible gives zeros, not NaN
    full = torch.full((Tq, Tk), float("-inf"), device=DEV)
    assert (rd.softmax(s, mask=full) == 0).all()
    pad = torch.zeros(B, 1, 1, Tk, device=DEV)
    pad[1, ..., -5:] = float("-inf")
    torch.testing.assert_close(rd.softmax(s, mask=pad), torch.softmax(s + pad, -1), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sum_axis_broadcast_permute(dtype):
    g = torch.Generator(device=DEV).manual_seed(8)
    x = torch.randn(5, 70, 9, 4, generator=g, device=DEV).to(dtype)
    for axis in range(4):
        torch.testing.assert_close(rd.sum_axis(x, axis), x.float().sum(axis), rtol=1e-4, atol=1e-3)
    long = torch.randn(3000, 24, generator=g, device=DEV).to(dtype)
    torch.testing.assert_close(rd.sum_axis(long, 0, 0.5), long.float().sum(0) * 0.5, rtol=1e-4, atol=1e-2)
    again = rd.sum_axis(long, 0, 0.5)
    assert torch.equal(again, rd.sum_axis(long, 0, 0.5))
    s = torch.randn(5, 9, generator=g, device=DEV)
    b = rd.broadcast_axis(s, 1, 6, dtype=dtype)
    torch.testing.assert_close(b.float(), s[:, None, :].expand(5, 6, 9).to(dtype).float())
    acc = torch.ones(5, 6, 9, device=DEV, dtype=dtype)
    rd.broadcast_axis(s, 1, 6, accumulate_into=acc)
    torch.testing.assert_close(acc.float(), (1 + s[:, None, :].expand(5, 6, 9)).to(dtype).float(), **_tol(dtype))
    for order in ([0, 1, 3, 2], [3, 1, 0, 2], [2, 3, 0, 1], [1, 0, 2, 3]):
        assert torch.equal(rd.permute(x, order), x.permute(order).contiguous())
    m = torch.randn(3, 45, 70, generator=g, device=DEV).to(dtype)
    assert torch.equal(rd.transpose(m), m.transpose(1, 2).contiguous())
    six = torch.randn(2, 3, 4, 5, 6, 7, generator=g, device=DEV).to(dtype)
    assert torch.equal(rd.permute(six, [5, 3, 1, 0, 2, 4]), six.permute(5, 3, 1, 0, 2, 4).contiguous())


def test_gather_one_hot_class_match():
    g = torch.Generator(device=DEV).manual_seed(9)
    table = torch.randn(50, 24, generator=g, device=DEV).bfloat16()
    ids = torch.tensor([[0, 49, 7], [3, -1, 50]], device=DEV)
    got = rd.gather_rows(table, ids)
    assert torch.equal(got[0], table[ids[0]]) and torch.equal(got[1, 0], table[3])
    assert (got[1, 1:] == 0).all()
    oh = rd.one_hot(torch.tensor([2, 0, 4], device=DEV), 5)
    assert torch.equal(oh, torch.eye(5, device=DEV)[[2, 0, 4]])
    logits = torch.randn(300, 1000, generator=g, device=DEV)
    logits[5, 10] = logits[5, 20] = 50.0                        # a tie: the lower index wins
    targets = logits.argmax(-1).to(torch.int32)
    targets[5] = 10
    targets[::3] = -1                                           # left out
    targets[1] = (targets[1] + 1) % 1000                        # a miss
    want = ((logits.argmax(-1) == targets) & (targets >= 0)).sum().item()
    assert rd.class_match(logits, targets).item() == want


@pytest.mark.parametrize("case", ["plain", "repeats", "long_targets", "impossible"])
def test_ctc_loss_and_gradient(case):
    g = torch.Generator(device=DEV).manual_seed(10)
    T, B, Cn, L = 50, 6, 12, 14
    logits = torch.randn(T, B, Cn, generator=g, device=DEV, requires_grad=True)
    targets = torch.randint(1, Cn, (B, L), generator=g, device=DEV)
    in_len = torch.tensor([50, 43, 50, 31, 29, 50], device=DEV)
    tg_len = torch.tensor([14, 9, 1, 7, 14, 0], device=DEV)
    if case == "repeats":
        targets[:, 1::2] = targets[:, 0::2]
    if case == "long_targets":
        T, L = 300, 140
        logits = torch.randn(T, B, Cn, generator=g, device=DEV, requires_grad=True)
        targets = torch.randint(1, Cn, (B, L), generator=g, device=DEV)
        in_len = torch.tensor([300, 290, 300, 281, 300, 300], device=DEV)
        tg_len = torch.tensor([140, 100, 1, 70, 139, 0], device=DEV)
    if case == "impossible":
        in_len[0] = 10                                           # 14 labels cannot fit 10 frames
    lp = torch.log_softmax(logits, -1)
    loss = ctc_ops.ctc_loss(lp, targets, in_len, tg_len)
    ref_logits = logits.detach().clone().requires_grad_(True)
    ref = ctc_ops.ctc_reference(torch.log_softmax(ref_logits, -1), targets, in_len, tg_len)
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-3)
    finite = torch.isfinite(ref)
    weights = torch.randn(B, generator=g, device=DEV)
    (loss[finite] * weights[finite]).sum().backward()
    (ref[finite] * weights[finite]).sum().backward()
    # a sequence without an alignment gets a zero gradient here (the library's is NaN there): compare the others
    torch.testing.assert_close(logits.grad[:, finite], ref_logits.grad[:, finite], rtol=1e-3, atol=1e-4)
    assert (logits.grad[:, ~finite] == 0).all()
    # reruns agree bit for bit
    l2 = ctc_ops.ctc_loss(torch.log_softmax(logits.detach(), -1), targets, in_len, tg_len)
    assert torch.equal(l2, loss.detach())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lstm_and_gru_cells(dtype):
    g = torch.Generator(device=DEV).manual_seed(11)
    B, H = 7, 96
    gates = torch.randn(B, 4 * H, generator=g, device=DEV).to(dtype).requires_grad_(True)
    c0 = torch.randn(B, H, generator=g, device=DEV).to(dtype).requires_grad_(True)
    h, c = rc.lstm_cell(gates, c0)
    gr, cr = gates.detach().float().requires_grad_(True), c0.detach().float().requires_grad_(True)
    hr, cr1 = rc.lstm_cell_reference(gr, cr)
    torch.testing.assert_close(h.float(), hr, **_tol(dtype))
    torch.testing.assert_close(c.float(), cr1, **_tol(dtype))
    dh, dc = (torch.randn(B, H, generator=g, device=DEV).to(dtype) for _ in range(2))
    torch.autograd.backward([h, c], [dh, dc])
    torch.autograd.backward([hr, cr1], [dh.float(), dc.float()])
    tol = dict(rtol=4e-2, atol=4e-2) if dtype == torch.bfloat16 else _tol(dtype)
    torch.testing.assert_close(gates.grad.float(), gr.grad, **tol)
    torch.testing.assert_close(c0.grad.float(), cr.grad, **tol)

    gi, gh = (torch.randn(B, 3 * H, generator=g, device=DEV).to(dtype).requires_grad_(True) for _ in range(2))
    h0 = torch.randn(B, H, generator=g, device=DEV).to(dtype).requires_grad_(True)
    h1 = rc.gru_cell(gi, gh, h0)
    refs = [t.detach().float().requires_grad_(True) for t in (gi, gh, h0)]
    h1r = rc.gru_cell_reference(*refs)
    torch.testing.assert_close(h1.float(), h1r, **_tol(dtype))
    h1.backward(dh)
    h1r.backward(dh.float())
    for mine, ref in zip((gi, gh, h0), refs):
        torch.testing.assert_close(mine.grad.float(), ref.grad, **tol)


@pytest.mark.parametrize("kind", ["lstm", "gru"])
def test_recurrent_module_matches_torch(kind, monkeypatch):
    torch.manual_seed(12)
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)        # the library module would round to tf32
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_tf32", False)
    cls = torch.nn.LSTM if kind == "lstm" else torch.nn.GRU
    m = cls(24, 40, num_layers=2, batch_first=True, bidirectional=True).to(DEV)
    x = torch.randn(5, 11, 24, device=DEV, requires_grad=True)
    out, state = rc.run_module(m, x)
    xr = x.detach().clone().requires_grad_(True)
    out_r, state_r = m(xr)
    torch.testing.assert_close(out, out_r, rtol=1e-4, atol=1e-4)
    hn = state[0] if kind == "lstm" else state
    hn_r = state_r[0] if kind == "lstm" else state_r
    torch.testing.assert_close(hn, hn_r, rtol=1e-4, atol=1e-4)
    w = torch.randn_like(out)
    grads = torch.autograd.grad((out * w).sum(), [x, m.weight_hh_l0, m.weight_ih_l1_reverse])
    grads_r = torch.autograd.grad((out_r * w).sum(), [xr, m.weight_hh_l0, m.weight_ih_l1_reverse])
    for a, b in zip(grads, grads_r):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("cfg", [dict(stride=1, padding=1, dilation=1), dict(stride=2, padding=0, dilation=1),
                                 dict(stride=(2, 1), padding=(2, 1), dilation=(2, 1))])
def test_conv2d_bf16_against_fp32(cfg):
    g = torch.Generator(device=DEV).manual_seed(13)
    N, Cc, H, W, OC, K = 3, 5, 19, 17, 12, 3
    x = torch.randn(N, Cc, H, W, generator=g, device=DEV).bfloat16().requires_grad_(True)
    w = (0.2 * torch.randn(OC, Cc, K, K, generator=g, device=DEV)).bfloat16().requires_grad_(True)
    b = torch.randn(OC, generator=g, device=DEV).bfloat16().requires_grad_(True)
    y = cv.conv2d(x, w, b, **cfg)
    refs = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = torch.nn.functional.conv2d(*refs, **cfg)
    assert y.shape == yr.shape
    torch.testing.assert_close(y.float(), yr, rtol=3e-2, atol=5e-2)
    dy = torch.randn(yr.shape, generator=g, device=DEV).bfloat16()
    y.backward(dy)
    yr.backward(dy.float())
    for mine, ref, tol in zip((x, w, b), refs, (0.08, 0.5, 0.5)):
        torch.testing.assert_close(mine.grad.float(), ref.grad, rtol=5e-2, atol=tol)


def test_conv1d_and_fp32_opt_in():
    g = torch.Generator(device=DEV).manual_seed(14)
    x = torch.randn(2, 8, 50, generator=g, device=DEV)
    w = 0.2 * torch.randn(16, 8, 5, generator=g, device=DEV)
    exact = cv.conv1d(x, w, None, 2, 2)                                        # fp32 stays with the library
    torch.testing.assert_close(exact, torch.nn.functional.conv1d(x, w, None, 2, 2), rtol=1e-4, atol=1e-4)
    mine = cv.conv1d(x, w, None, 2, 2, allow_bf16_products=True)
    torch.testing.assert_close(mine, exact, rtol=3e-2, atol=5e-2)
    assert not torch.equal(mine, exact)                                        # the products really were bf16


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_depthwise_and_pooling(dtype):
    g = torch.Generator(device=DEV).manual_seed(15)
    N, Cc, H, W = 2, 6, 15, 14
    tol = dict(rtol=3e-2, atol=6e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    x = torch.randn(N, Cc, H, W, generator=g, device=DEV).to(dtype).requires_grad_(True)
    w = (0.3 * torch.randn(Cc, 1, 3, 3, generator=g, device=DEV)).to(dtype).requires_grad_(True)
    b = torch.randn(Cc, generator=g, device=DEV).to(dtype).requires_grad_(True)
    y = cv.conv2d(x, w, b, stride=2, padding=1, groups=Cc)
    refs = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = torch.nn.functional.conv2d(*refs, stride=2, padding=1, groups=Cc)
    torch.testing.assert_close(y.float(), yr, **tol)
    dy = torch.randn(yr.shape, generator=g, device=DEV).to(dtype)
    y.backward(dy)
    yr.backward(dy.float())
    for mine, ref in zip((x, w, b), refs):
        torch.testing.assert_close(mine.grad.float(), ref.grad, rtol=3e-2, atol=0.15 if dtype == torch.bfloat16 else 1e-4)

    for kw in (dict(kernel=2), dict(kernel=3, stride=2, padding=1), dict(kernel=(3, 2), stride=(1, 2), ceil_mode=True)):
        xa = x.detach().clone().requires_grad_(True)
        xb = x.detach().clone().requires_grad_(True)
        p = cv.max_pool2d(xa, **kw)
        pr = torch.nn.functional.max_pool2d(xb, kw["kernel"], kw.get("stride"), kw.get("padding", 0),
                                            ceil_mode=kw.get("ceil_mode", False))
        assert torch.equal(p, pr)
        dp = torch.randn(pr.shape, generator=g, device=DEV).to(dtype)
        p.backward(dp)
        pr.backward(dp)
        torch.testing.assert_close(xa.grad.float(), xb.grad.float(), **tol)
    for include in (True, False):
        xa = x.detach().clone().requires_grad_(True)
        xb = x.detach().clone().requires_grad_(True)
        p = cv.avg_pool2d(xa, 3, 2, 1, count_include_pad=include)
        pr = torch.nn.functional.avg_pool2d(xb, 3, 2, 1, count_include_pad=include)
        torch.testing.assert_close(p.float(), pr.float(), **tol)
        dp = torch.randn(pr.shape, generator=g, device=DEV).to(dtype)
        p.backward(dp)
        pr.backward(dp)
        torch.testing.assert_close(xa.grad.float(), xb.grad.float(), **tol)
