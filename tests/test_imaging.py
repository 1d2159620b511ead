"""Imaging on the CPU: resampling and warps against Pillow byte for byte, coverage against two oracles, the TrueType
reader against FreeType's rendering, codecs against Pillow's readers, effects for determinism."""
import io

import numpy as np
import pytest
import torch

PIL = pytest.importorskip("PIL")
from PIL import Image, ImageDraw, ImageFilter, ImageFont  # noqa: E402

from idrak_b200 import imaging as im  # noqa: E402
from idrak_b200.imaging import warp as W  # noqa: E402

PIL_FILTERS = {"box": Image.BOX, "bilinear": Image.BILINEAR, "hamming": Image.HAMMING, "bicubic": Image.BICUBIC,
               "lanczos": Image.LANCZOS}


def _font():
    f = ImageFont.load_default(size=40)
    if not hasattr(f, "font_bytes"):
        pytest.skip("this Pillow has no embedded TrueType font")
    return f, im.TrueTypeFont(f.font_bytes)


@pytest.mark.parametrize("name", sorted(PIL_FILTERS))
def test_resize_matches_pillow_exactly(name):
    rng = np.random.default_rng(0)
    for (h, w, c, mode) in [(37, 53, 3, "RGB"), (64, 48, 1, "L"), (50, 40, 4, "CMYK")]:
        a = rng.integers(0, 256, (h, w, c), dtype=np.uint8)
        pil = Image.fromarray(a[..., 0] if c == 1 else a, mode)
        for (oh, ow) in [(20, 31), (90, 120), (h, 2 * w), (h // 3, w)]:
            ref = np.asarray(pil.resize((ow, oh), PIL_FILTERS[name])).reshape(oh, ow, c)
            got = im.resize(torch.from_numpy(a), (oh, ow), name).numpy()
            assert np.array_equal(ref, got), (name, (h, w, c), (oh, ow))


def test_resize_box_argument_and_float_images():
    rng = np.random.default_rng(1)
    a = rng.integers(0, 256, (60, 70, 3), dtype=np.uint8)
    box = (3.5, 2.25, 60.0, 50.5)
    ref = np.asarray(Image.fromarray(a).resize((33, 29), Image.BICUBIC, box=box))
    assert np.array_equal(ref, im.resize(torch.from_numpy(a), (29, 33), "bicubic", box=box).numpy())
    f = rng.random((40, 50)).astype(np.float32)
    ref = np.asarray(Image.fromarray(f, mode="F").resize((77, 23), Image.LANCZOS))
    assert np.allclose(ref, im.resize(torch.from_numpy(f), (23, 77), "lanczos").numpy(), atol=1e-6)
    with pytest.raises(ValueError):
        im.resize(torch.from_numpy(a), (10, 10), "nope")


def test_warp_matches_pillow_transform_exactly():
    rng = np.random.default_rng(2)
    a = rng.integers(0, 256, (40, 50, 3), dtype=np.uint8)
    pil = Image.fromarray(a)
    coef = im.rotation(17.0, 50, 40)
    for name, r in (("nearest", Image.NEAREST), ("bilinear", Image.BILINEAR), ("bicubic", Image.BICUBIC)):
        ref = np.asarray(pil.transform((50, 40), Image.PERSPECTIVE, tuple(coef), resample=r, fillcolor=(9, 8, 7)))
        assert np.array_equal(ref, im.warp(torch.from_numpy(a), coef, mode=name, fill=(9, 8, 7)).numpy()), name
    assert np.array_equal(np.asarray(pil.rotate(17.0, resample=Image.BILINEAR)), im.warp(torch.from_numpy(a), coef).numpy())
    pc = im.quad_to_quad([(0, 0), (50, 0), (50, 40), (0, 40)], [(3, 2), (47, 5), (44, 38), (1, 35)])
    ref = np.asarray(pil.transform((60, 45), Image.PERSPECTIVE, tuple(pc), resample=Image.BILINEAR))
    assert np.array_equal(ref, im.warp(torch.from_numpy(a), pc, size=(45, 60)).numpy())


def test_rank_and_blur_filters():
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (30, 36, 3), dtype=np.uint8)
    pil, x = Image.fromarray(a), torch.from_numpy(a)[None]
    for flt, got in ((ImageFilter.MedianFilter(3), im.median_filter(x, 3)), (ImageFilter.MinFilter(3), im.min_filter(x, 3)),
                     (ImageFilter.MaxFilter(5), im.max_filter(x, 5))):
        ref = np.asarray(pil.filter(flt))
        assert np.array_equal(ref[2:-2, 2:-2], got[0].numpy()[2:-2, 2:-2])
    ref = np.asarray(pil.filter(ImageFilter.BoxBlur(2))).astype(int)
    assert np.abs(ref[2:-2, 2:-2] - im.box_blur(x, 2)[0].numpy().astype(int)[2:-2, 2:-2]).max() <= 1
    flat = torch.full((1, 20, 20, 1), 77, dtype=torch.uint8)
    assert (im.gaussian_blur(flat, 2.0) == 77).all()
    spot = torch.zeros(1, 41, 41, 1, dtype=torch.uint8)
    spot[0, 20, 20] = 255
    g = im.gaussian_blur(spot, 3.0)[0, :, :, 0].float()
    ys = torch.arange(41.0) - 20
    var = (g.sum(1) * ys * ys).sum() / g.sum()
    assert 6.0 < var.item() < 12.5             # a box cascade of variance ~ sigma^2 = 9 (8-bit rounding loses the tails)


def test_coverage_is_the_exact_area():
    p = im.Path().move_to(2.3, 2.1).line_to(30.7, 4.2).quad_to(40, 20, 20.5, 30.25).line_to(5, 25).close()
    cov = im.coverage_reference([p], 48, 40)[0]
    segs = p.flatten().astype(np.float64)
    shoelace = 0.5 * abs(sum(x0 * y1 - x1 * y0 for x0, y0, x1, y1 in segs))
    assert abs(cov.sum() - shoelace) < 1e-9
    ss = im.supersample_reference(p, 48, 40, 16)
    assert np.abs(cov - ss).max() < 0.03
    # a square with a hole wound the other way; the same outline under both fill rules
    q = im.Path().move_to(-5, -5).line_to(20, -5).line_to(20, 20).line_to(-5, 20)
    q.move_to(5, 5).line_to(5, 15).line_to(15, 15).line_to(15, 5)
    assert abs(im.coverage_reference([q], 30, 30)[0].sum() - 300.0) < 1e-9          # clipped at the left / top edges
    assert abs(im.coverage_reference([q], 30, 30, rule="evenodd")[0].sum() - 300.0) < 1e-9
    # overlapping squares wound the same way: non-zero fills the union, even-odd leaves the overlap empty
    o = im.Path().move_to(2, 2).line_to(12, 2).line_to(12, 12).line_to(2, 12)
    o.move_to(7, 7).line_to(17, 7).line_to(17, 17).line_to(7, 17)
    assert abs(im.coverage_reference([o], 20, 20)[0].sum() - 175.0) < 1e-9
    assert abs(im.coverage_reference([o], 20, 20, rule="evenodd")[0].sum() - 150.0) < 1e-9
    e = im.coverage_reference([im.ellipse(20, 20, 15, 10)], 40, 40)[0]
    assert abs(e.sum() - np.pi * 150) / (np.pi * 150) < 2e-3
    t = im.Path().move_to(25.5, 25.5).line_to(40, 26).line_to(30, 45)             # runs off the right and bottom
    assert np.abs(im.coverage_reference([t], 30, 30)[0] - im.supersample_reference(t, 30, 30, 16)).max() < 0.03
    m = im.rasterize([p, q], 48, 40)
    assert m.dtype == torch.uint8 and m.shape == (2, 40, 48) and m.max() == 255


def test_truetype_outlines_agree_with_freetype():
    pil_font, font = _font()
    assert font.units_per_em > 0 and font.num_glyphs > 50 and font.glyph_index(ord("A")) > 0
    assert font.glyph_index(0x10FFFF) == 0
    text = "Idrak B200 &gy"
    ascent = font.ascender * 40 / font.units_per_em
    # single glyphs (FreeType rounds advances to whole pixels, so a line of text drifts); hinting still moves stems
    # by fractions of a pixel: compare lightly blurred ink, and the total ink
    for ch in "B&g8Q":
        mask = im.render_text(font, ch, 40, padding=4)
        H, Wd = mask.shape
        ref = Image.new("L", (Wd, H), 0)
        ImageDraw.Draw(ref).text((4, 4 + ascent), ch, font=pil_font, fill=255, anchor="ls")
        ref_t = torch.from_numpy(np.asarray(ref).copy())
        blur = lambda t: im.box_blur(t[None, :, :, None], 1)[0, :, :, 0].double().numpy()
        ours, theirs = blur(mask), blur(ref_t)
        corr = np.corrcoef(ours.ravel(), theirs.ravel())[0, 1]
        assert corr > 0.93, (ch, corr)
        assert abs(ours.sum() - theirs.sum()) / theirs.sum() < 0.1, ch
    w, asc, desc = font.measure(text, 40)
    assert abs(w - pil_font.getlength(text)) < 0.06 * w and asc > desc > 0


def test_page_layout_boxes_and_alignment():
    _, font = _font()
    text = "the quick brown fox jumps over the lazy dog " * 6 + "\n\nsecond paragraph here"
    page = im.compose_page(font, text, 400, 300, font_size=18, margins=(20, 20, 20, 20), align="justify")
    assert page.image.shape == (300, 400, 1) and page.image.dtype == torch.uint8
    assert page.image.min() < 60 and page.image.max() == 245
    assert len(page.lines) > 4 and "" in page.lines
    first_line = [w for w in page.words if w.line == 0]
    assert abs(first_line[0].x0 - 20) < 1e-6 and abs(first_line[-1].x1 - 380) < 1.0           # justified to both margins
    for w in page.words:                                                              # ink sits inside its word box
        box = page.image[int(w.y0): int(np.ceil(w.y1)), int(w.x0): int(np.ceil(w.x1)), 0]
        assert box.min() < 200, w
    outside = page.image[:, :18, 0]
    assert (outside == 245).all()
    right = im.compose_page(font, "a few words", 300, 80, font_size=18, margins=(10, 10, 10, 10), align="right")
    assert abs(right.words[-1].x1 - 290) < 1e-6
    assert im.wrap(font, "averyveryverylongwordthatdoesnotfit next", 18, 50) == [["averyveryverylongwordthatdoesnotfit"], ["next"]]


def test_codecs_round_trip_and_read_pillow_files():
    rng = np.random.default_rng(4)
    for shape, mode in (((23, 31), "L"), ((23, 31, 3), "RGB"), ((9, 14, 4), "RGBA"), ((9, 14, 2), "LA")):
        a = rng.integers(0, 256, shape, dtype=np.uint8)
        a[:5] = 7                                               # flat rows: the 'up' and 'sub' filters win somewhere
        data = im.encode_png(a)
        assert np.array_equal(im.decode(data), a)
        assert np.array_equal(np.asarray(Image.open(io.BytesIO(data))), a)          # Pillow reads what we write
        buf = io.BytesIO()
        Image.fromarray(a, mode).save(buf, "PNG")
        assert np.array_equal(im.decode_png(buf.getvalue()), a)                       # and we read what Pillow writes
    pal = Image.fromarray(rng.integers(0, 256, (12, 17, 3), dtype=np.uint8)).quantize(16)
    buf = io.BytesIO()
    pal.save(buf, "PNG")
    assert np.array_equal(im.decode(buf.getvalue()), np.asarray(pal.convert("RGB")))
    bits = Image.fromarray((rng.random((10, 13)) > 0.5).astype(np.uint8) * 255).convert("1")
    buf = io.BytesIO()
    bits.save(buf, "PNG")
    assert np.array_equal(im.decode(buf.getvalue()), np.asarray(bits.convert("L")))
    for shape in ((11, 15), (11, 15, 3)):
        a = rng.integers(0, 256, shape, dtype=np.uint8)
        for fmt in ("bmp", "ppm"):
            data = im.encode(a, fmt)
            assert np.array_equal(im.decode(data), a), (shape, fmt)
            assert np.array_equal(np.asarray(Image.open(io.BytesIO(data))), a)
    assert np.array_equal(im.decode_pnm(b"P2\n# c\n3 2\n15\n0 5 15\n15 5 0\n"), np.array([[0, 85, 255], [255, 85, 0]], np.uint8))
    bad = bytearray(im.encode_png(np.zeros((4, 4), np.uint8)))
    bad[40] ^= 1
    with pytest.raises(im.ImageFormatError):
        im.decode(bytes(bad))
    with pytest.raises(im.ImageFormatError):
        im.decode(b"GIF89a")


def test_effects_are_seeded_and_change_the_page():
    _, font = _font()
    page = im.compose_page(font, "effects on a page of text " * 8, 256, 192, font_size=16, margins=(12, 12, 12, 12)).image
    rgb = page.expand(-1, -1, 3).contiguous()[None]
    assert len(im.EFFECTS) >= 35
    for name in sorted(im.EFFECTS):
        a = im.apply(rgb, [name], seed=5, strength=0.8)
        b = im.apply(rgb, [name], seed=5, strength=0.8)
        assert a.shape == rgb.shape and a.dtype == torch.uint8, name
        assert torch.equal(a, b), name
        assert not torch.equal(a, rgb), name
    a = im.random_pipeline(rgb, seed=3, count=5)
    assert torch.equal(a, im.random_pipeline(rgb, seed=3, count=5))
    assert not torch.equal(a, im.random_pipeline(rgb, seed=4, count=5))
    with pytest.raises(KeyError):
        im.apply(rgb, ["nope"])
    # the noise has the statistics it claims
    flat = torch.full((1, 128, 128, 1), 128, dtype=torch.uint8)
    n = im.pixel_pass(flat, im.PixelPass(noise_sigma=0.05, seed=9)).float()
    assert abs(n.mean().item() - 128) < 0.5 and abs(n.std().item() - 0.05 * 255) < 0.6
    sp = im.pixel_pass(flat, im.PixelPass(salt=0.02, pepper=0.03, seed=9))
    assert abs((sp == 255).float().mean().item() - 0.02) < 0.005 and abs((sp == 0).float().mean().item() - 0.03) < 0.005


def test_baseline_jpeg_decoder_against_libjpeg():
    yy, xx = np.mgrid[0:67, 0:93]
    img = np.stack([(np.sin(xx / 9) + 1) * 120, (np.cos(yy / 7) + 1) * 110, (xx + yy) % 256], -1).astype(np.uint8)

    def both(array, **save):
        buf = io.BytesIO()
        Image.fromarray(array).save(buf, "JPEG", **save)
        mine = im.decode(buf.getvalue()).astype(int)
        ref = Image.open(io.BytesIO(buf.getvalue()))
        return mine, np.asarray(ref if array.ndim == 2 else ref.convert("RGB")).astype(int)

    mine, ref = both(img[..., 0], quality=75)
    assert np.array_equal(mine, ref)                                     # grey: the inverse DCT alone
    mine, ref = both(img, quality=90, subsampling=0)
    assert mine.shape == (67, 93, 3) and np.abs(mine - ref).max() <= 2    # colour conversion rounding
    mine, ref = both(img, quality=85, subsampling=0, restart_marker_blocks=3)
    assert np.abs(mine - ref).max() <= 2
    for sub in (1, 2):                                                    # chroma replicated here, interpolated there
        mine, ref = both(img, quality=90, subsampling=sub)
        assert np.abs(mine - ref).mean() < 4.0
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, "JPEG", progressive=True)
    with pytest.raises(im.ImageFormatError, match="progressive"):
        im.decode(buf.getvalue())


def test_jpeg_encoder_round_trips_and_an_independent_decoder_reads_it():
    import io

    import numpy as np

    from idrak_b200.imaging import codecs
    from idrak_b200.imaging.jpeg import _canonical, _code_lengths, decode_jpeg, encode_jpeg
    rng = np.random.default_rng(0)
    y, x = np.mgrid[0:70, 0:93]
    img = np.stack([128 + 100 * np.sin(x / 9.0) * np.cos(y / 7.0), (x * 2.5) % 256, (y * 3 + x) % 256], -1)
    img = (img + rng.normal(0, 3, img.shape)).clip(0, 255).astype(np.uint8)

    def psnr(a, b):
        return 10 * np.log10(255 ** 2 / ((a.astype(float) - b.astype(float)) ** 2).mean())

    sizes = {}
    for quality, sub, floor in ((95, False, 37.0), (75, False, 33.0), (50, True, 27.0)):
        data = encode_jpeg(img, quality, sub)
        back = decode_jpeg(data)
        assert back.shape == img.shape and psnr(img, back) > floor, (quality, psnr(img, back))
        sizes[quality] = len(data)
    assert sizes[95] > sizes[75] > sizes[50]
    grey = encode_jpeg(img[..., 0], 85)
    assert decode_jpeg(grey).shape == (70, 93) and psnr(img[..., 0], decode_jpeg(grey)) > 36
    assert codecs.decode(codecs.encode(img, "jpeg")).shape == img.shape
    try:
        from PIL import Image
    except ImportError:
        Image = None
    if Image is not None:                       # a decoder that shares no code with this package reads the file
        seen = np.array(Image.open(io.BytesIO(encode_jpeg(img, 90))).convert("RGB"))
        assert psnr(img, seen) > 35
    # code lengths: never longer than 16 bits, a prefix code with one code point to spare (Kraft sum below one)
    freq = {s: 2 ** min(s, 40) for s in range(60)}
    lengths = _code_lengths(freq)
    assert max(lengths.values()) <= 16 and sum(2.0 ** -v for v in lengths.values()) < 1.0
    counts, symbols, codes = _canonical(lengths)
    assert sum(counts) == len(symbols) == 60 and all(code < (1 << n) - 1 or n < max(lengths.values()) for code, n in codes.values())
    assert _code_lengths({7: 10}) == {7: 1}
