"""8-bit-moment AdamW: the maps round-trip, the CPU statement tracks fp32 AdamW closely, state is 4x smaller;
on a GPU the kernel matches the CPU statement."""
import pytest
import torch

from idrak_b200.ops.optim8 import Adam8bit, signed_code, signed_value, unsigned_code, unsigned_value


def test_maps_are_monotone_and_round_trip():
    codes = torch.arange(256, dtype=torch.uint8)
    sv, uv = signed_value(codes), unsigned_value(codes)
    assert torch.all(sv[1:] > sv[:-1]) and torch.all(uv[1:] > uv[:-1]) and sv[0] == -1 and sv[-1] == 1 and uv[-1] == 1
    assert torch.equal(signed_code(sv), codes) and torch.equal(unsigned_code(uv), codes)
    assert int(unsigned_code(torch.tensor([1e-9]))[0]) == 1          # a tiny second moment never becomes zero


def _problem(device, dtype=torch.float32):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(1000, device=device, dtype=dtype) * 0.1)
    x = torch.randn(64, 1000, device=device)
    y = x @ torch.randn(1000, device=device) * 0.05
    return w, x, y


def test_tracks_fp32_adamw_on_cpu():
    w8, x, y = _problem("cpu")
    w32 = torch.nn.Parameter(w8.detach().clone())
    o8 = Adam8bit([w8], lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    o32 = torch.optim.AdamW([w32], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    first = None
    for _ in range(60):
        for w, o in ((w8, o8), (w32, o32)):
            o.zero_grad()
            loss = ((x @ w - y) ** 2).mean()
            loss.backward()
            if o is o32:
                torch.nn.utils.clip_grad_norm_([w32], 1.0)
            o.step()
        first = first if first is not None else float(loss.detach())
    l8, l32 = float(((x @ w8 - y) ** 2).mean()), float(((x @ w32 - y) ** 2).mean())
    assert l8 < 0.01 * first and l32 < 0.01 * first              # both solve the problem
    assert (w8 - w32).abs().max() < 0.05
    assert o8.state_bytes() < 0.27 * (2 * 4 * w8.numel())
    again = Adam8bit([torch.nn.Parameter(w8.detach().clone())], lr=1e-2)
    again.load_state_dict(o8.state_dict())
    assert again.step_count == 60 and torch.equal(again.m8[0], o8.m8[0])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernel_matches_cpu_statement(dtype):
    wc, x, y = _problem("cpu")
    wg = torch.nn.Parameter(wc.detach().clone().cuda().to(dtype))
    if dtype == torch.bfloat16:
        wc = torch.nn.Parameter(wg.detach().float().cpu())
    oc = Adam8bit([wc], lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    og = Adam8bit([wg], lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(3)
    for _ in range(5):
        grad = torch.randn(1000, generator=g) * 0.3
        wc.grad = grad.clone()
        wg.grad = grad.cuda().to(dtype)
        if dtype == torch.bfloat16:
            wc.grad = wg.grad.float().cpu()
        oc.step()
        og.step()
    torch.testing.assert_close(og.master[0].cpu(), oc.master[0], rtol=1e-4, atol=2e-5)
    assert (og.m8[0].cpu().int() - oc.m8[0].int()).abs().max() <= 1 and (og.v8[0].cpu().int() - oc.v8[0].int()).abs().max() <= 1
    torch.testing.assert_close(og.m_absmax[0].cpu(), oc.m_absmax[0], rtol=1e-4, atol=1e-7)
