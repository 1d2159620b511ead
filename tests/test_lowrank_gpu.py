"""The low-rank term contracted inside the base product: kernel against fp32, and the adapter path that uses it against
the separate-product path."""
import pytest
import torch

from idrak_b200.ops.gemm import gemm_lowrank, gemm_lowrank_reference, lowrank_linear

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(g, *shape, scale=1.0):
    return (scale * torch.randn(*shape, generator=g, device=DEV)).bfloat16()


@pytest.mark.parametrize("M,N,K,R", [(256, 512, 256, 16), (1000, 384, 520, 48), (128, 128, 64, 8), (513, 1032, 4096, 64),
                                     (300, 264, 192, 136)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_lowrank_product_against_fp32(M, N, K, R, b_mn):
    g = torch.Generator(device=DEV).manual_seed(M + R)
    a, a2 = _rand(g, M, K), _rand(g, M, R)
    b = _rand(g, K, N, scale=0.05) if b_mn else _rand(g, N, K, scale=0.05)
    b2 = _rand(g, R, N, scale=0.2) if b_mn else _rand(g, N, R, scale=0.2)
    bias, res = _rand(g, N), _rand(g, M, N)
    got = gemm_lowrank(a, b, a2, b2, b_mn=b_mn, bias=bias, residual=res)
    want = gemm_lowrank_reference(a, b, a2, b2, b_mn=b_mn, bias=bias, residual=res)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=3e-2)
    plain = gemm_lowrank(a, b, a2, b2, b_mn=b_mn)
    # the second pair really is in the sum
    base_only = gemm_lowrank_reference(a, b, torch.zeros_like(a2), b2, b_mn=b_mn)
    assert (plain.float() - base_only.float()).abs().max() > 0.5
    assert torch.equal(plain, gemm_lowrank(a, b, a2, b2, b_mn=b_mn))


def test_lowrank_linear_gradients():
    g = torch.Generator(device=DEV).manual_seed(5)
    M, K, N, R = 384, 256, 320, 32
    x = _rand(g, 3, M // 3, K).requires_grad_(True)
    w = _rand(g, N, K, scale=0.05).requires_grad_(True)
    bias = _rand(g, N).requires_grad_(True)
    res = _rand(g, 3, M // 3, N).requires_grad_(True)
    A = _rand(g, R, K, scale=0.1).requires_grad_(True)
    B = _rand(g, N, R, scale=0.1).requires_grad_(True)
    y = lowrank_linear(x, w, bias, res, A, B)
    refs = [t.detach().float().requires_grad_(True) for t in (x, w, bias, res, A, B)]
    xr, wr, br, rr, Ar, Br = refs
    yr = xr @ wr.t() + (xr @ Ar.t()) @ Br.t() + br + rr
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=3e-2)
    dy = _rand(g, 3, M // 3, N, scale=0.1)
    y.backward(dy)
    yr.backward(dy.float())
    for mine, ref, tol in zip((x, w, bias, res, A, B), refs, (0.02, 0.08, 0.08, 0.0, 0.08, 0.08)):
        torch.testing.assert_close(mine.grad.float(), ref.grad, rtol=5e-2, atol=tol + 1e-3)


@pytest.mark.parametrize("quant", [None, "int4"])
def test_adapters_ride_in_the_base_product(quant, monkeypatch):
    from idrak_b200.adapters import lora
    from idrak_b200.adapters.lora import AdapterSet, LoraAdapter, project_with_adapters
    g = torch.Generator(device=DEV).manual_seed(7)
    K, dq, dkv = 256, 256, 64
    N = dq + 2 * dkv
    x = _rand(g, 2, 300, K).requires_grad_(True)
    w = _rand(g, N, K, scale=0.05)
    bias = _rand(g, N)
    slices = {"q": (0, dq), "k": (dq, dq + dkv), "v": (dq + dkv, N)}
    ads = AdapterSet()
    for name, (lo, hi) in slices.items():
        if name == "k":
            continue                                        # one slice without an adapter
        ad = LoraAdapter(K, hi - lo, rank=16, alpha=32.0, dtype=torch.bfloat16, device=DEV)
        with torch.no_grad():
            ad.B.copy_(_rand(g, hi - lo, 16, scale=0.1))
        ads.items[name] = ad
    packed = None
    if quant:
        from idrak_b200.quant.weights import quantize_weight
        packed = quantize_weight(w.t().contiguous().float(), quant).to(DEV)

    dy = _rand(g, 2, 300, N, scale=0.1)

    def run(fused: bool):
        if not fused:
            monkeypatch.setattr(lora, "_stacked_adapters", lambda *a, **k: None)
        else:
            monkeypatch.undo()
        for p in list(ads.parameters()) + [x]:
            p.grad = None
        y = project_with_adapters(x, w, bias, ads, slices, packed=packed)
        y.backward(dy)
        return y.detach(), x.grad.clone(), [p.grad.clone() for p in ads.parameters()]

    y1, dx1, g1 = run(True)
    y0, dx0, g0 = run(False)
    torch.testing.assert_close(y1.float(), y0.float(), rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(dx1.float(), dx0.float(), rtol=5e-2, atol=2e-2)
    for a, b in zip(g1, g0):
        torch.testing.assert_close(a.float(), b.float(), rtol=5e-2, atol=0.3)
        assert a.float().abs().max() > 1.0                      # the comparison is not vacuous
