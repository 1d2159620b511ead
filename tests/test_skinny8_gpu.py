"""The int8-weight few-row kernel against the de-quantised product in fp32."""
import pytest
import torch

from idrak_b200.ops.skinny import skinny8_linear, skinny8_reference
from idrak_b200.quant import Int8Weight, qgemm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(g, *shape, scale=1.0):
    return (scale * torch.randn(*shape, generator=g, device=DEV)).bfloat16()


@pytest.mark.parametrize("M", [1, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(4096, 4096), (768, 4096), (4096, 512), (1000, 1040), (136, 64)])
def test_plain_product(M, N, K):
    g = torch.Generator(device=DEV).manual_seed(M + N)
    w8 = Int8Weight.quantize(torch.randn(K, N, generator=g, device=DEV) * 0.05)
    x = _rand(g, M, K)
    got = skinny8_linear(x, w8)
    want = skinny8_reference(x, w8)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(got, skinny8_linear(x, w8))               # fixed reduction order: reruns agree bit for bit


def test_bias_residual_and_output_buffer():
    g = torch.Generator(device=DEV).manual_seed(3)
    M, N, K = 40, 2048, 1536
    w8 = Int8Weight.quantize(torch.randn(K, N, generator=g, device=DEV) * 0.05)
    x, bias, res = _rand(g, M, K), _rand(g, N), _rand(g, M, N)
    buf = torch.zeros(64, N, dtype=torch.bfloat16, device=DEV)
    got = skinny8_linear(x, w8, bias, res, out=buf[:M])
    assert got.data_ptr() == buf.data_ptr() and (buf[M:] == 0).all()
    torch.testing.assert_close(got.float(), skinny8_reference(x, w8, bias, res).float(), rtol=2e-2, atol=3e-2)
    # the packed-weight product routes few rows here and agrees with the unpack-first path
    from idrak_b200.quant import weights
    via_qgemm = qgemm(x, w8, bias=bias, residual=res)
    assert torch.equal(via_qgemm, got)


@pytest.mark.parametrize("gate", ["silu", "gelu"])
@pytest.mark.parametrize("ff", [1792, 3584, 200])
def test_gated_pair(gate, ff):
    g = torch.Generator(device=DEV).manual_seed(ff)
    M, K = 64, 1024
    w8 = Int8Weight.quantize(torch.randn(K, 2 * ff, generator=g, device=DEV) * 0.05)
    x, bias = _rand(g, M, K), _rand(g, 2 * ff, scale=0.1)
    got = skinny8_linear(x, w8, bias, gate=gate)
    want = skinny8_reference(x, w8, bias, gate=gate)
    assert got.shape == (M, ff)
    torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)
