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


MODES = [  # B, S, H, Hkv, D, window, spans, softcap
    (2, 512, 4, 4, 64, 128, None, None),
    (1, 640, 4, 2, 128, 200, None, None),
    (2, 512, 4, 4, 64, None, [(0, 100), (100, 384), (384, 400), (400, 512)], None),
    (1, 1000, 2, 1, 128, None, [(0, 7), (7, 530), (530, 1000)], None),
    (1, 384, 4, 4, 64, None, None, 30.0),
    (1, 384, 2, 2, 128, 96, [(0, 130), (130, 384)], 50.0),
]


@pytest.mark.parametrize("B,S,H,Hkv,D,window,spans,softcap", MODES)
def test_flash_window_packed_sequences_and_softcap(B, S, H, Hkv, D, window, spans, softcap):
    """Sliding window, sequences packed into one row (a lower key bound per position) and tanh soft-capping run inside
    the attention kernels, forward and backward; the oracle is the fp32 statement with explicit masks."""
    q, k, v = (_rand((B, S, H, D), 1).requires_grad_(), _rand((B, S, Hkv, D), 2).requires_grad_(),
               _rand((B, S, Hkv, D), 3).requires_grad_())
    row_start = ops.row_starts_from_spans(spans, B, S, "cuda") if spans else None
    out = ops.attention(q, k, v, True, None, window, row_start, softcap)
    do = _rand(out.shape, 4)
    out.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = ops.attention_reference(qr, kr, vr, True, None, window, row_start, softcap)
    ref.backward(do.float())
    _close(out, ref, 2e-2)
    _close(q.grad, qr.grad, 5e-2)
    _close(k.grad, kr.grad, 5e-2)
    _close(v.grad, vr.grad, 5e-2)


def test_packed_row_equals_the_sequences_run_one_by_one():
    """One launch over a packed row gives each sequence what a launch of its own gives (the same tiles of scores are
    masked instead of skipped, so the results agree to the rounding of the running maximum)."""
    B, S, H, D = 1, 768, 4, 64
    spans = [(0, 200), (200, 201), (201, 640), (640, 768)]
    q, k, v = _rand((B, S, H, D), 1), _rand((B, S, H, D), 2), _rand((B, S, H, D), 3)
    packed, _ = ops.flash_forward(q, k, v, True, None, None, ops.row_starts_from_spans(spans, B, S, "cuda"))
    for lo, hi in spans:
        alone, _ = ops.flash_forward(q[:, lo:hi].contiguous(), k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), True)
        _close(packed[:, lo:hi], alone, 1e-2)
