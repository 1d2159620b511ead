"""Host statements of the element-wise, reduction, CTC, recurrent and convolution operations (what a CPU tensor runs and
what the device kernels are compared with)."""
import pytest
import torch

from idrak_b200.ops import conv as cv
from idrak_b200.ops import ctc as ctc_ops
from idrak_b200.ops import pointwise as pw
from idrak_b200.ops import recurrent as rc
from idrak_b200.ops import reduce as rd


def test_unary_and_binary_names_cover_the_kernel_tables():
    x = torch.linspace(0.5, 2.0, 16)
    for name in pw.UNARY:
        y = pw.unary(name, x, 0.5, 1.5)
        assert y.shape == x.shape and torch.isfinite(y).all(), name
    for name in pw.BINARY:
        assert pw.binary(name, x, x + 1).shape == x.shape
    with pytest.raises(KeyError, match="unknown unary"):
        pw.unary("cbrt", x)
    with pytest.raises(KeyError, match="unknown binary"):
        pw.binary("xor", x, x)
    torch.testing.assert_close(pw.unary_backward("square", x, torch.ones_like(x)), 2 * x)
    acc = torch.ones_like(x)
    pw.unary_backward("exp", x, torch.ones_like(x), accumulate_into=acc)
    torch.testing.assert_close(acc, 1 + x.exp())
    torch.testing.assert_close(pw.clamp(x, high=1.0), x.clamp(max=1.0))
    torch.testing.assert_close(pw.axpby(2.0, x, -1.0, x), x)


def test_dropout_generator_is_a_function_of_seed_and_index():
    u = pw.uniform_reference(99, 2000)
    assert torch.equal(u, pw.uniform_reference(99, 2000))
    assert not torch.equal(u, pw.uniform_reference(100, 2000))
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean().item() - 0.5) < 0.03
    x = torch.ones(2000)
    y = pw.dropout(x, 0.5, 99)
    assert set(y.unique().tolist()) == {0.0, 2.0}
    assert torch.equal(y, pw.dropout(x, 0.5, 99))
    with pytest.raises(ValueError):
        pw.dropout(x, 1.0, 1)


def test_softmax_cpu_forms():
    s = torch.randn(2, 3, 5, 8)
    causal = rd.scale_mask_softmax(s, 0.5, None, causal=True)
    keep = torch.ones(5, 8, dtype=torch.bool).tril(3)
    want = torch.softmax((0.5 * s).masked_fill(~keep, float("-inf")), -1)
    torch.testing.assert_close(causal, want)
    assert (rd.softmax(s, mask=torch.full((5, 8), float("-inf"))) == 0).all()
    torch.testing.assert_close(rd.log_softmax(s, 1), torch.log_softmax(s, 1))
    torch.testing.assert_close(rd.sum_axis(s, 2, 0.2), s.sum(2) * 0.2)
    assert torch.equal(rd.permute(s, [3, 0, 2, 1]), s.permute(3, 0, 2, 1).contiguous())
    with pytest.raises(ValueError, match="not a permutation"):
        rd.permute(s, [0, 0, 1, 2])
    assert rd.class_match(torch.eye(4), torch.tensor([0, 1, 3, -1])).item() == 2
    assert torch.equal(rd.one_hot(torch.tensor([1, 5]), 3), torch.tensor([[0., 1., 0.], [0., 0., 0.]]))
    got = rd.gather_rows(torch.arange(6.0).reshape(3, 2), torch.tensor([2, 7]))
    assert torch.equal(got, torch.tensor([[4., 5.], [0., 0.]]))


def test_ctc_cpu_path_is_per_sequence():
    lp = torch.log_softmax(torch.randn(12, 2, 5), -1)
    loss = ctc_ops.ctc_loss(lp, torch.tensor([[1, 2, 3], [4, 4, 0]]), torch.tensor([12, 12]), torch.tensor([3, 2]))
    assert loss.shape == (2,) and torch.isfinite(loss).all()
    with pytest.raises(ValueError):
        ctc_ops.ctc_loss(lp[0], torch.tensor([[1]]), torch.tensor([1]), torch.tensor([1]))


@pytest.mark.parametrize("kind", ["lstm", "gru"])
def test_recurrent_drivers_follow_torch_modules(kind):
    torch.manual_seed(0)
    cls = torch.nn.LSTM if kind == "lstm" else torch.nn.GRU
    m = cls(6, 10, num_layers=2, bidirectional=True, batch_first=True)
    x = torch.randn(3, 7, 6)
    out, state = rc.run_module(m, x)
    out_r, state_r = m(x)
    torch.testing.assert_close(out, out_r, rtol=1e-5, atol=1e-6)
    if kind == "lstm":
        torch.testing.assert_close(state[1], state_r[1], rtol=1e-5, atol=1e-6)
    else:
        torch.testing.assert_close(state, state_r, rtol=1e-5, atol=1e-6)


def test_output_sizes_follow_the_library():
    x = torch.randn(1, 2, 11, 13)
    for k, s, p, ceil in ((3, 2, 1, False), (3, 2, 1, True), (2, 2, 0, True), (3, 3, 1, True), (5, 4, 2, True)):
        want = torch.nn.functional.max_pool2d(x, k, s, p, ceil_mode=ceil).shape
        assert (cv._out_size(11, k, s, p, 1, ceil), cv._out_size(13, k, s, p, 1, ceil)) == tuple(want[-2:])
    assert torch.equal(cv.max_pool2d(x, 2), torch.nn.functional.max_pool2d(x, 2))
    w = torch.randn(4, 2, 3, 3)
    torch.testing.assert_close(cv.conv2d(x, w, None, 2, 1), torch.nn.functional.conv2d(x, w, None, 2, 1))
    torch.testing.assert_close(cv.conv1d(x[:, :, 0], w[:, :, 0], None, 1, 1),
                               torch.nn.functional.conv1d(x[:, :, 0], w[:, :, 0], None, 1, 1))
