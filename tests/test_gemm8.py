"""fp8 (e4m3) quantisers and the 8-bit tensor-core product against a plain PyTorch fp32 statement."""
import warnings

import pytest
import torch

from idrak_b200.ops.gemm8 import (E4M3_MAX, Float8Rows, dequantize_rows, gemm8, gemm8_reference, linear_fp8,
                                  quantize_rows, quantize_rows_reference)


def test_row_quantiser_reference_properties():
    x = torch.randn(9, 64) * torch.logspace(-3, 3, 9)[:, None]
    x[4] = 0
    q = quantize_rows_reference(x)
    assert q.codes.dtype == torch.uint8 and q.codes.shape == x.shape and q.scales.shape == (9,)
    assert q.scales[4].item() == 1.0                               # an all-zero row keeps scale 1
    back = dequantize_rows(q, torch.float32)
    # e4m3 has 3 mantissa bits: relative error of a normal value is at most 2^-4
    big = x.abs() > x.abs().amax(1, keepdim=True) * 2 ** -6
    assert ((back - x).abs()[big] <= x.abs()[big] * 2 ** -4 + 1e-12).all()
    assert torch.allclose(back.abs().amax(1)[[0, 8]], x.abs().amax(1)[[0, 8]], rtol=1e-6)   # the row maximum is exact


def test_gemm8_cpu_statement_and_linear():
    x, w = torch.randn(6, 48), torch.randn(10, 48)
    a, b = quantize_rows(x.bfloat16()), quantize_rows(w.bfloat16())
    y = gemm8(a, b, bias=torch.ones(10, dtype=torch.bfloat16))
    ref = x @ w.t() + 1
    assert (y.float() - ref).abs().max().item() < 0.12 * ref.abs().max().item()
    assert linear_fp8(x.bfloat16().reshape(2, 3, 48), b).shape == (2, 3, 10)


def test_float8_scope_says_what_it_runs():
    from idrak_b200 import core
    from idrak_b200.core import scopes
    before = scopes.fallbacks["float8_to_bfloat16"]
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        with core.mixed_precision("float8"):
            assert core.product_precision() == "bfloat16"
    assert scopes.fallbacks["float8_to_bfloat16"] == before + 1
    assert any("float8" in str(w.message) for w in seen)


def _rand(shape, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,K", [(7, 64), (300, 768), (129, 4096), (33, 8192), (5, 16384)])
def test_row_quantiser_kernel(rows, K):
    x = _rand((rows, K), 3.0, 1)
    x[rows // 2] = 0
    q = quantize_rows(x)
    ref = quantize_rows_reference(x)
    assert torch.allclose(q.scales, ref.scales.to(q.scales.device), rtol=1e-6)
    # round-to-nearest of the same quotient: codes equal the plain statement's, except that a quotient on a rounding
    # boundary may fall to the neighbouring code where the two divide differently (one step, a fraction of a percent)
    a, b = q.codes.to(torch.int16), ref.codes.to(q.codes.device).to(torch.int16)
    mag_a, mag_b = a & 0x7F, b & 0x7F
    assert ((mag_a - mag_b).abs() <= 1).all()
    assert ((a & 0x80) == (b & 0x80))[(mag_a > 0) & (mag_b > 0)].all()
    assert (mag_a != mag_b).float().mean().item() < 5e-3
    got = dequantize_rows(q).float()
    assert (got.abs().amax(1) <= x.float().abs().amax(1) * (1 + 2 ** -7)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 256), (1024, 2304, 768), (200, 136, 80),
                                   (4096, 768, 3072), (130, 1000, 1040), (64, 64, 16)])
def test_gemm8_kernel_matches_statement(M, N, K):
    a, b = quantize_rows(_rand((M, K), 1.0, 2)), quantize_rows(_rand((N, K), 0.1, 3))
    bias = _rand((N,), 1.0, 4)
    for bi in (None, bias):
        out = gemm8(a, b, bi)
        ref = gemm8_reference(a, b, bi)
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= 1e-2 * (ref.float().abs().max().item() + 1e-6), (err, bi is not None)
    assert torch.equal(gemm8(a, b), gemm8(a, b))
    from idrak_b200 import _native
    torch.cuda.synchronize()
    _native.check_status("gemm8")


@pytest.mark.gpu
def test_linear_fp8_tracks_the_bf16_product():
    x, w = _rand((512, 1024), 1.0, 5), _rand((768, 1024), 0.05, 6)
    y8 = linear_fp8(x, w).float()
    y16 = (x.float() @ w.float().t())
    rel = (y8 - y16).norm() / y16.norm()
    assert rel.item() < 0.06, rel.item()
