"""tcgen05 GEMM against a plain PyTorch fp32 statement of the same contract."""
import pytest
import torch

from idrak_b200.ops import gemm, gemm_reference, linear

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _check(out, ref, tol=2e-2):
    out, ref = out.float(), ref.float()
    err = (out - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"max err {err} vs scale {denom}"


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 768), (1024, 2304, 768), (200, 136, 72), (64, 64, 64),
          (130, 100, 1000), (4096, 768, 3072), (128, 50304, 768)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_majors(M, N, K, a_mn, b_mn):
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("leading dimension must be a multiple of 8")
    a = _rand((K, M) if a_mn else (M, K), 1.0, 1)
    b = _rand((K, N) if b_mn else (N, K), 1.0, 2)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, splits=1)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _check(out, ref)


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_gemm_splitk_matches_and_is_deterministic(splits):
    M, N, K = 768, 768, 4096
    a, b = _rand((K, M), 1.0, 3), _rand((K, N), 1.0, 4)
    ref = gemm_reference(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    o1 = gemm(a, b, a_mn=True, b_mn=True, splits=splits, out_dtype=torch.float32)
    o2 = gemm(a, b, a_mn=True, b_mn=True, splits=splits, out_dtype=torch.float32)
    _check(o1, ref, 5e-3)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("M", [1, 7, 16, 32, 33, 48, 64])
@pytest.mark.parametrize("N,K,splits", [(512, 256, 1), (6144, 4096, None), (4096, 1024, 4), (1000, 520, 1)])
def test_gemm_few_rows(M, N, K, splits):
    """Decode-sized products take the few-row layout (part of the A tile per stage, more stages): every epilogue the
    serving path uses, with and without split-K, and N / K that are not tile multiples."""
    a, b = _rand((M, K), 1.0, 11), _rand((N, K), 0.05, 12)
    bias, res = _rand((N,), 1.0, 13), _rand((M, N), 1.0, 14)
    _check(gemm(a, b, splits=splits), gemm_reference(a, b, out_dtype=torch.float32))
    _check(gemm(a, b, bias=bias, residual=res, splits=splits),
           gemm_reference(a, b, bias=bias, residual=res, out_dtype=torch.float32))
    out, pre = gemm(a, b, bias=bias, act="gelu", splits=splits)
    ref, ref_pre = gemm_reference(a, b, bias=bias, act="gelu", out_dtype=torch.float32)
    _check(pre, ref_pre)
    _check(out, ref)
    o32 = gemm(a, b, splits=splits, out_dtype=torch.float32)
    assert torch.equal(o32, gemm(a, b, splits=splits, out_dtype=torch.float32))
    _check(o32, gemm_reference(a, b, out_dtype=torch.float32), 5e-3)


def test_gemm_epilogues():
    M, N, K = 512, 1024, 256
    a, b = _rand((M, K), 1.0, 5), _rand((N, K), 0.1, 6)
    bias, res = _rand((N,), 1.0, 7), _rand((M, N), 1.0, 8)
    out = gemm(a, b, bias=bias, residual=res)
    _check(out, gemm_reference(a, b, bias=bias, residual=res, out_dtype=torch.float32))
    out, pre = gemm(a, b, bias=bias, act="gelu")
    ref, ref_pre = gemm_reference(a, b, bias=bias, act="gelu", out_dtype=torch.float32)
    _check(pre, ref_pre)
    _check(out, ref)
    g = gemm(a, b, act="gelu_grad", aux=pre)
    _check(g, gemm_reference(a, b, act="gelu_grad", aux=pre, out_dtype=torch.float32))
    # the training pair: activation and derivative out of the forward epilogue, one multiply in the backward one
    out_d, dact = gemm(a, b, bias=bias, act="gelu_d")
    ref_d, ref_dact = gemm_reference(a, b, bias=bias, act="gelu_d", out_dtype=torch.float32)
    _check(out_d, ref_d)
    _check(dact, ref_dact)
    _check(gemm(a, b, act="mul_aux", aux=dact), gemm_reference(a, b, act="mul_aux", aux=dact, out_dtype=torch.float32))
    acc = torch.ones((M, N), dtype=torch.float32, device="cuda")
    gemm(a, b, out=acc, beta=True, alpha=0.5)
    _check(acc, gemm_reference(a, b, alpha=0.5, out_dtype=torch.float32) + 1.0)


def test_linear_autograd_matches_torch():
    x = _rand((4, 96, 256), 1.0, 9).requires_grad_()
    w = _rand((384, 256), 0.05, 10).requires_grad_()
    b = _rand((384,), 0.1, 11).requires_grad_()
    y = linear(x, w, b)
    dy = _rand(y.shape, 1.0, 12)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    _check(y, yr)
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    _check(b.grad, br.grad)


def test_autotune_measures_once_and_keeps_results_equal(tmp_path):
    from idrak_b200 import config
    from idrak_b200.runtime import reset_tuner, tuner
    config.settings.set("IDRAK_AUTOTUNE", True)
    config.settings.set("IDRAK_TUNING_CACHE", str(tmp_path / "tuning.json"))
    reset_tuner()
    try:
        a, b = _rand((48, 2048), 1.0, 21), _rand((1536, 2048), 0.05, 22)
        first = gemm(a, b)
        t = tuner()
        assert t.measured == 1 and any(k.startswith("gemm.splits:64x1536x2048") for k in t.entries())
        second = gemm(a, b)
        assert t.measured == 1
        ref = gemm_reference(a, b, out_dtype=torch.float32)
        _check(first, ref)
        _check(second, ref)
    finally:
        config.settings._overrides.pop("IDRAK_AUTOTUNE", None)
        config.settings._overrides.pop("IDRAK_TUNING_CACHE", None)
        reset_tuner()


def _pair_case(M, N, K, a_mn, b_mn):
    a = _rand((K, M) if a_mn else (M, K), 1.0, 31)
    b = _rand((K, N) if b_mn else (N, K), 0.05, 32)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, splits=1)
    _check(out, ref)
    assert torch.equal(out, gemm(a, b, a_mn=a_mn, b_mn=b_mn, splits=1))
    if not a_mn and not b_mn:
        bias, res = _rand((N,), 1.0, 33), _rand((M, N), 1.0, 34)
        _check(gemm(a, b, bias=bias, residual=res, splits=1), gemm_reference(a, b, bias=bias, residual=res, out_dtype=torch.float32))
        o, pre = gemm(a, b, bias=bias, act="gelu", splits=1)
        r, r_pre = gemm_reference(a, b, bias=bias, act="gelu", out_dtype=torch.float32)
        _check(pre, r_pre)
        _check(o, r)
        _check(gemm(a, b, act="gelu_grad", aux=pre, splits=1), gemm_reference(a, b, act="gelu_grad", aux=pre, out_dtype=torch.float32))
        o, dact = gemm(a, b, bias=bias, act="gelu_d", splits=1)
        r, r_dact = gemm_reference(a, b, bias=bias, act="gelu_d", out_dtype=torch.float32)
        _check(dact, r_dact)
        _check(o, r)
        _check(gemm(a, b, act="mul_aux", aux=dact, splits=1), gemm_reference(a, b, act="mul_aux", aux=dact, out_dtype=torch.float32))
        acc = torch.ones((M, N), dtype=torch.float32, device="cuda")
        gemm(a, b, out=acc, beta=True, alpha=0.5, splits=1)
        _check(acc, gemm_reference(a, b, alpha=0.5, out_dtype=torch.float32) + 1.0)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(2048, 2304, 768), (4096, 768, 3072), (1504, 1000, 520), (16384, 768, 768)])
def test_gemm_large_products(M, N, K, a_mn, b_mn):
    """Products large enough for the CTA-pair kernel (256 x 256 tiles on two SMs; IDRAK_GEMM_PAIR=2 sends every such
    product there, the default only the shapes where it measured faster, 0 none): all operand layouts, sizes that are
    not tile multiples, every epilogue."""
    _pair_case(M, N, K, a_mn, b_mn)
    from idrak_b200 import _native
    _native.check_status("large products")
