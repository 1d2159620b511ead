"""De-quant-fused int8 / int4 GEMM vs the de-quantised matrix in fp32."""
import pytest
import torch

from idrak_b200.quant import Int4Weight, Int8Weight, dequantize_bf16, qgemm, qlinear

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("cls", [Int8Weight, Int4Weight])
@pytest.mark.parametrize("M,K,N", [(256, 512, 768), (130, 200, 136), (8, 1024, 1024), (1024, 4096, 512)])
def test_qgemm_forward_and_transposed(cls, M, K, N):
    w = _rand((K, N), 0.05, 1).float()
    qw = cls.quantize(w)
    deq = qw.dequantize()
    assert (dequantize_bf16(qw).float() - deq).abs().max().item() <= 2e-2 * deq.abs().max().item()
    x = _rand((M, K), 1.0, 2)
    y = qgemm(x, qw)
    ref = x.float() @ deq
    assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-3
    dy = _rand((M, N), 1.0, 3)
    dx = qgemm(dy, qw, transposed=True)
    refx = dy.float() @ deq.t()
    assert (dx.float() - refx).abs().max().item() < 2e-2 * refx.abs().max().item() + 1e-3


def test_qlinear_autograd_and_epilogue():
    K, N = 512, 384
    qw = Int4Weight.quantize(_rand((K, N), 0.05, 1).float())
    x = _rand((2, 64, K), 1.0, 2).requires_grad_()
    b, r = _rand((N,), 0.1, 3), _rand((2, 64, N), 1.0, 4)
    y = qlinear(x, qw, b, r)
    dy = _rand(y.shape, 1.0, 5)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = xr @ qw.dequantize() + b.float() + r.float()
    yr.backward(dy.float())
    assert (y.float() - yr).abs().max().item() < 2e-2 * yr.abs().max().item()
    assert (x.grad.float() - xr.grad).abs().max().item() < 2e-2 * xr.grad.abs().max().item()


def test_many_rows_take_the_dense_path_and_agree_with_the_fused_kernel(monkeypatch):
    from idrak_b200.quant import weights
    qw = Int4Weight.quantize(_rand((1024, 768), 0.05, 1).float())
    x, bias = _rand((2048, 1024), 1.0, 2), _rand((768,), 0.1, 3)
    dense = qgemm(x, qw, bias=bias)
    monkeypatch.setattr(weights, "DENSE_ROWS", 1 << 30)
    fused = qgemm(x, qw, bias=bias)
    ref = x.float() @ qw.dequantize() + bias.float()
    for y in (dense, fused):
        assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    assert (dense.float() - fused.float()).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("cls", [Int8Weight, Int4Weight])
def test_few_rows_unpack_first_and_agree_with_the_fused_kernel(cls, monkeypatch):
    from idrak_b200.quant import weights
    qw = cls.quantize(_rand((1024, 768), 0.05, 1).float())
    x = _rand((16, 1024), 1.0, 2)
    unpacked = qgemm(x, qw)
    monkeypatch.setattr(weights, "FEW_ROWS", 0)
    fused = qgemm(x, qw)
    ref = x.float() @ qw.dequantize()
    for y in (unpacked, fused):
        assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
