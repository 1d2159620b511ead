"""The raster / resampling / warp / filter / effect kernels against their CPU restatements (which the CPU tests pin to
Pillow and to the analytic area)."""
import numpy as np
import pytest
import torch

from idrak_b200 import imaging as im

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return "cuda"


def test_resize_kernel_is_byte_exact(dev):
    rng = np.random.default_rng(0)
    a = torch.from_numpy(rng.integers(0, 256, (3, 97, 131, 3), dtype=np.uint8))
    for name in im.FILTERS:
        for size in ((40, 50), (200, 300), (97, 262), (31, 131)):
            ref = im.resize(a, size, name)
            got = im.resize(a.to(dev), size, name)
            assert torch.equal(ref, got.cpu()), (name, size)
    ref = im.resize(a, (55, 66), "bicubic", box=(3.5, 2.25, 120.0, 90.5))
    assert torch.equal(ref, im.resize(a.to(dev), (55, 66), "bicubic", box=(3.5, 2.25, 120.0, 90.5)).cpu())
    f = torch.from_numpy(rng.random((2, 64, 80, 1)).astype(np.float32))
    assert torch.allclose(im.resize(f, (33, 150), "lanczos"), im.resize(f.to(dev), (33, 150), "lanczos").cpu(), atol=1e-5)


def test_coverage_kernel_matches_the_area_oracle(dev):
    rng = np.random.default_rng(1)
    paths = [im.Path().move_to(2.3, 2.1).line_to(30.7, 4.2).quad_to(40, 20, 20.5, 30.25).line_to(5, 25),
             im.ellipse(24, 20, 30, 12),                                      # clipped left and right
             im.Path().move_to(-5, -5).line_to(20, -5).line_to(20, 20).line_to(-5, 20)
                      .move_to(5, 5).line_to(5, 15).line_to(15, 15).line_to(15, 5)]
    star = im.Path()
    pts = [(24 + 18 * np.cos(2 * np.pi * (2 * i) / 5), 20 + 18 * np.sin(2 * np.pi * (2 * i) / 5)) for i in range(5)]
    star.move_to(*pts[0])
    for p in pts[1:]:
        star.line_to(*p)
    paths.append(star)                                                        # self-intersecting: the rules differ
    for _ in range(4):
        p = im.Path().move_to(*rng.uniform(-10, 58, 2))
        for _ in range(6):
            p.cubic_to(*rng.uniform(-10, 58, 6))
        paths.append(p)
    for rule in ("nonzero", "evenodd"):
        ref = im.coverage_reference(paths, 48, 40, rule)
        got = im.rasterize(paths, 48, 40, rule, device=dev, dtype=torch.float32).cpu().numpy()
        assert np.abs(ref - got).max() < 2e-4, rule
        u8 = im.rasterize(paths, 48, 40, rule, device=dev).cpu().numpy().astype(int)
        assert np.abs(np.rint(ref * 255) - u8).max() <= 1
    assert im.rasterize([], 8, 8, device=dev).shape == (0, 8, 8)
    assert int(im.rasterize([im.Path()], 8, 8, device=dev).sum()) == 0


def test_text_page_on_the_device_equals_the_cpu_page(dev):
    from PIL import ImageFont
    f = ImageFont.load_default(size=20)
    if not hasattr(f, "font_bytes"):
        pytest.skip("this Pillow has no embedded TrueType font")
    font = im.TrueTypeFont(f.font_bytes)
    text = "pages are rasterised in one launch " * 12
    cpu = im.compose_page(font, text, 500, 360, font_size=20, margins=(20, 20, 20, 20))
    gpu = im.compose_page(font, text, 500, 360, font_size=20, margins=(20, 20, 20, 20), device=dev)
    d = (cpu.image.int() - gpu.image.cpu().int()).abs()
    assert d.max() <= 1 and (d > 0).float().mean() < 0.01
    assert cpu.image.min() < 60


def test_warp_and_filter_kernels_equal_the_cpu_path(dev):
    rng = np.random.default_rng(2)
    a = torch.from_numpy(rng.integers(0, 256, (2, 60, 75, 3), dtype=np.uint8))
    coefs = np.stack([im.rotation(11.0, 75, 60), im.quad_to_quad([(0, 0), (75, 0), (75, 60), (0, 60)],
                                                                [(4, 3), (70, 6), (66, 57), (2, 52)])])
    for mode in ("nearest", "bilinear", "bicubic"):
        ref = im.warp(a, coefs, size=(64, 80), mode=mode, fill=(200, 100, 50))
        got = im.warp(a.to(dev), coefs, size=(64, 80), mode=mode, fill=(200, 100, 50)).cpu()
        assert torch.equal(ref, got), mode
    f = a.float() / 255
    assert torch.allclose(im.warp(f, coefs, mode="bicubic"), im.warp(f.to(dev), coefs, mode="bicubic").cpu(), atol=1e-5)
    assert torch.equal(im.box_blur(a, 3, 1), im.box_blur(a.to(dev), 3, 1).cpu())
    for size, rank in ((3, 0), (3, 4), (5, 24), (5, 7)):
        assert torch.equal(im.rank_filter(a, size, rank), im.rank_filter(a.to(dev), size, rank).cpu()), (size, rank)
    assert torch.equal(im.gaussian_blur(a, 2.5), im.gaussian_blur(a.to(dev), 2.5).cpu())


def test_effect_kernel_matches_its_restatement(dev):
    rng = np.random.default_rng(3)
    a = torch.from_numpy(rng.integers(0, 256, (2, 70, 90, 3), dtype=np.uint8))
    p = im.PixelPass(gain=0.9, bias=0.03, gamma=1.3, grad_x=0.2, grad_y=-0.3, vignette=0.4, vignette_power=2.5,
                     noise_sigma=0.05, salt=0.01, pepper=0.02, fibre=0.2, fibre_scale=0.2, grey_noise=False, seed=1234567)
    ref = im.pixel_pass(a, p).int()
    got = im.pixel_pass(a.to(dev), p).cpu().int()
    d = (ref - got).abs()
    assert d.max() <= 2 and (d > 0).float().mean() < 0.05            # fast-math transcendentals move a few values by one
    for name in sorted(im.EFFECTS):
        out = im.apply(a.to(dev), [name], seed=5, strength=0.8)
        assert out.is_cuda and out.shape == a.shape and out.dtype == torch.uint8, name
        assert torch.equal(out, im.apply(a.to(dev), [name], seed=5, strength=0.8)), name
    big = torch.from_numpy(rng.integers(0, 256, (4, 1024, 768, 3), dtype=np.uint8)).to(dev)
    out = im.random_pipeline(big, seed=1, count=6)
    assert out.shape == big.shape
