"""Image kernels against torch.nn.functional on the same inputs (forward and backward)."""
import pytest
import torch
import torch.nn.functional as F

from idrak_b200.ops import image as I

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["bilinear", "nearest"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_resize_normalize(mode, dtype):
    g = torch.Generator().manual_seed(0)
    img = torch.randint(0, 256, (3, 37, 53, 3), generator=g, dtype=torch.uint8)
    mean, std = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
    want = I.resize_normalize(img, (24, 40), mean, std, mode)                       # CPU statement
    got = I.resize_normalize(img.cuda(), (24, 40), mean, std, mode, dtype=dtype)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(got.float().cpu(), want, rtol=tol, atol=tol)
    up = I.resize_normalize(img.cuda(), (80, 120), mean, std, mode)
    torch.testing.assert_close(up.cpu(), I.resize_normalize(img, (80, 120), mean, std, mode), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("mode", ["nearest", "bilinear"])
@pytest.mark.parametrize("shape,size", [((2, 3, 17, 23), (34, 46)), ((2, 3, 32, 40), (13, 9)), ((1, 2, 8, 8), (8, 8)),
                                        ((1, 1, 5, 7), (16, 3))])
def test_interpolate_forward_backward(mode, shape, size):
    x = torch.randn(*shape, device="cuda", requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    y = I.interpolate(x, size, mode)
    yr = F.interpolate(xr, size=size, mode=mode, **({"align_corners": False} if mode == "bilinear" else {}))
    torch.testing.assert_close(y, yr, rtol=1e-5, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-4, atol=1e-4)
    yb = I.interpolate(x.detach().bfloat16(), size, mode)
    torch.testing.assert_close(yb.float(), yr.detach(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kind", ["avg", "max"])
@pytest.mark.parametrize("shape,size", [((2, 4, 14, 14), (7, 7)), ((2, 3, 15, 11), (4, 6)), ((1, 2, 6, 6), (1, 1)),
                                        ((1, 2, 5, 5), (7, 9))])
def test_adaptive_pools_forward_backward(kind, shape, size):
    x = torch.randn(*shape, device="cuda", requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    if kind == "avg":
        y, yr = I.adaptive_avg_pool(x, size), F.adaptive_avg_pool2d(xr, size)
    else:
        y, yr = I.adaptive_max_pool(x, size), F.adaptive_max_pool2d(xr, size)
    torch.testing.assert_close(y, yr, rtol=1e-5, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-5, atol=1e-5)
