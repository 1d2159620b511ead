"""tcgen05 flash attention forward/backward vs fp32 softmax(QK^T)V."""
import pytest
import torch

from idrak_b200 import ops

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol, f"err {err}"


CASES = [  # B, Sq, Skv, H, Hkv, D, causal
    (1, 128, 128, 1, 1, 64, False),
    (1, 128, 128, 1, 1, 64, True),
    (2, 256, 256, 4, 4, 64, True),
    (2, 1024, 1024, 12, 12, 64, True),
    (1, 384, 384, 8, 2, 128, True),
    (1, 200, 200, 2, 2, 64, True),
    (1, 100, 333, 4, 1, 128, False),
    (1, 128, 512, 2, 2, 64, True),
]


@pytest.mark.parametrize("B,Sq,Skv,H,Hkv,D,causal", CASES)
def test_flash_forward(B, Sq, Skv, H, Hkv, D, causal):
    q, k, v = _rand((B, Sq, H, D), 1), _rand((B, Skv, Hkv, D), 2), _rand((B, Skv, Hkv, D), 3)
    out, lse = ops.flash_forward(q, k, v, causal)
    ref = ops.attention_reference(q.float(), k.float(), v.float(), causal)
    _close(out, ref, 2e-2)


def test_flash_forward_from_fused_qkv_buffer():
    B, S, H, D = 2, 256, 4, 64
    qkv = _rand((B, S, 3 * H * D), 5)
    q, k, v = (qkv[..., i * H * D:(i + 1) * H * D].unflatten(-1, (H, D)) for i in range(3))
    out, _ = ops.flash_forward(q, k, v, True)
    _close(out, ops.attention_reference(q.float(), k.float(), v.float(), True), 2e-2)


@pytest.mark.parametrize("B,Sq,Skv,H,Hkv,D,causal", CASES)
def test_flash_backward(B, Sq, Skv, H, Hkv, D, causal):
    q, k, v = (_rand((B, Sq, H, D), 1).requires_grad_(), _rand((B, Skv, Hkv, D), 2).requires_grad_(),
               _rand((B, Skv, Hkv, D), 3).requires_grad_())
    out = ops.attention(q, k, v, causal)
    do = _rand(out.shape, 4)
    out.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = ops.attention_reference(qr, kr, vr, causal)
    ref.backward(do.float())
    _close(q.grad, qr.grad, 5e-2)
    _close(k.grad, kr.grad, 5e-2)
    _close(v.grad, vr.grad, 5e-2)
