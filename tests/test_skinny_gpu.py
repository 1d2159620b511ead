"""The few-row projection kernel (cluster split-K, fused epilogues) against the fp32 statement."""
import pytest
import torch

from idrak_b200.ops import skinny

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2):
    scale = max(1.0, b.float().abs().max().item())
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol * scale, f"{err} > {tol * scale}"


SHAPES = [  # M, N, K  (cluster sizes 8, 4, 1, 8, 1 on a 148-SM part; odd sizes exercise the masks)
    (64, 4096, 4096), (64, 6144, 4096), (64, 8192, 1024), (64, 4096, 14336), (64, 50304, 768),
    (1, 4096, 4096), (7, 1000, 520), (16, 128, 64), (17, 136, 72), (33, 2048, 2048), (48, 3000, 4096),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_plain_product_with_bias_and_residual(M, N, K):
    x, w = _rand((M, K), 1.0, 1), _rand((N, K), K ** -0.5, 2)
    b, r = _rand((N,), 0.5, 3), _rand((M, N), 1.0, 4)
    assert skinny.supported(x, w)
    _close(skinny.skinny_linear(x, w), skinny.skinny_reference(x, w))
    _close(skinny.skinny_linear(x, w, b, r), skinny.skinny_reference(x, w, b, r))


@pytest.mark.parametrize("M,ff,K,kind", [(64, 14336, 4096, "silu"), (64, 1792, 4096, "silu"), (5, 200, 512, "gelu"),
                                         (32, 4096, 1024, "relu"), (64, 64, 4096, "silu")])
def test_gated_pair_is_activated_inside_the_launch(M, ff, K, kind):
    x, w = _rand((M, K), 1.0, 1), _rand((2 * ff, K), K ** -0.5, 2)
    assert skinny.supported(x, w, kind)
    _close(skinny.skinny_linear(x, w, gate=kind), skinny.skinny_reference(x, w, gate=kind))
    b = _rand((2 * ff,), 0.3, 3)
    _close(skinny.skinny_linear(x, w, b, gate=kind), skinny.skinny_reference(x, w, b, gate=kind))


@pytest.mark.parametrize("M,N,K,gate", [(64, 6144, 4096, None), (9, 512, 2048, None), (64, 1024, 4096, "silu")])
def test_folded_rms_norm_equals_norm_then_product(M, N, K, gate):
    x = _rand((M, K), 2.0, 1)
    nw = (_rand((K,), 0.2, 5).float() + 1).to(torch.bfloat16)
    rows = 2 * N if gate else N
    w = _rand((rows, K), K ** -0.5, 2)
    folded = skinny.fold_norm(w, nw)
    got = skinny.skinny_linear(x, folded, gate=gate, norm_eps=1e-5)
    xf = x.float()
    normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
    want = skinny.skinny_reference(normed.to(torch.bfloat16), w, gate=gate)
    _close(got, want, 3e-2)


def test_result_is_the_same_bits_on_every_run_and_strided_inputs_work():
    x_full, w = _rand((64, 8192), 1.0, 1), _rand((4096, 4096), 0.02, 2)
    x = x_full[:, 4096:]                                  # a column slice: row stride 8192
    a = skinny.skinny_linear(x, w)
    for _ in range(3):
        assert torch.equal(a, skinny.skinny_linear(x, w))
    _close(a, skinny.skinny_reference(x, w))
    out = torch.zeros(64, 8192, dtype=torch.bfloat16, device="cuda")
    skinny.skinny_linear(x, w, out=out[:, :4096])
    assert torch.equal(out[:, :4096], a) and float(out[:, 4096:].abs().sum()) == 0.0
    torch.cuda.synchronize()
    from idrak_b200 import _native
    _native.check_status("skinny")
