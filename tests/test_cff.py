"""CFF outlines (``imaging/cff.py``) on a font assembled here byte by byte: every path operator family, hints and masks,
local and global subroutines, flex, the leading width - and the font class reading an ``OTTO`` file."""
import struct

import pytest
import torch

from idrak_b200 import imaging as im
from idrak_b200.imaging.cff import CffError, CffTable, read_dict, read_index


def num(n):
    if isinstance(n, float) and n != int(n):
        return b"\xff" + struct.pack(">i", int(round(n * 65536)))
    n = int(n)
    if -107 <= n <= 107:
        return bytes([n + 139])
    if 108 <= n <= 1131:
        n -= 108
        return bytes([247 + (n >> 8), n & 255])
    if -1131 <= n <= -108:
        n = -n - 108
        return bytes([251 + (n >> 8), n & 255])
    return b"\x1c" + struct.pack(">h", n)


def cs(*items):
    """Numbers and operator names -> charstring bytes."""
    ops = {"hstem": 1, "vstem": 3, "vmoveto": 4, "rlineto": 5, "hlineto": 6, "vlineto": 7, "rrcurveto": 8, "callsubr": 10,
           "return": 11, "endchar": 14, "hstemhm": 18, "hintmask": 19, "rmoveto": 21, "hmoveto": 22, "vstemhm": 23,
           "rcurveline": 24, "rlinecurve": 25, "vvcurveto": 26, "hhcurveto": 27, "callgsubr": 29, "vhcurveto": 30,
           "hvcurveto": 31, "hflex": (12, 34), "flex": (12, 35), "hflex1": (12, 36), "flex1": (12, 37), "sqrt": (12, 26)}
    out = b""
    for it in items:
        if isinstance(it, bytes):
            out += it
        elif isinstance(it, str):
            op = ops[it]
            out += bytes(op) if isinstance(op, tuple) else bytes([op])
        else:
            out += num(it)
    return out


def index(objects):
    if not objects:
        return b"\x00\x00"
    offs, at = [1], 1
    for o in objects:
        at += len(o)
        offs.append(at)
    size = 1 if at < 256 else 2
    return struct.pack(">HB", len(objects), size) + b"".join(o.to_bytes(size, "big") for o in offs) + b"".join(objects)


def int32(n):
    return b"\x1d" + struct.pack(">i", n)


def build_cff(charstrings, subrs=(), gsubrs=()):
    header = bytes([1, 0, 4, 1])
    names, strings, gsub = index([b"Test"]), index([]), index(list(gsubrs))
    top_len = 5 + 1 + 10 + 1                                   # int32 17 | int32 int32 18
    top_index_len = len(index([b"\x00" * top_len]))
    chars_at = len(header) + len(names) + top_index_len + len(strings) + len(gsub)
    chars = index(list(charstrings))
    private = num(500) + bytes([20]) + num(600) + bytes([21])
    private += num(len(private) + 2) + bytes([19])             # local subroutines right behind the dictionary
    top = int32(chars_at) + bytes([17]) + int32(len(private)) + int32(chars_at + len(chars)) + bytes([18])
    assert len(top) == top_len
    return header + names + index([top]) + strings + gsub + chars + private + index(list(subrs))


def build_otf(cff, cmap, advances, upem=1000):
    n = len(advances)
    head = bytearray(54)
    struct.pack_into(">H", head, 18, upem)
    maxp = struct.pack(">IH", 0x00005000, n)
    hhea = bytearray(36)
    struct.pack_into(">hhh", hhea, 4, 800, -200, 0)
    struct.pack_into(">H", hhea, 34, n)
    hmtx = b"".join(struct.pack(">Hh", a, 0) for a in advances)
    groups = b"".join(struct.pack(">III", c, c, g) for c, g in sorted(cmap.items()))
    sub = struct.pack(">HHIII", 12, 0, 16 + len(groups), 0, len(cmap)) + groups
    cm = struct.pack(">HHHHI", 0, 1, 3, 10, 12) + sub
    tables = {b"CFF ": cff, b"cmap": cm, b"head": bytes(head), b"hhea": bytes(hhea), b"hmtx": hmtx, b"maxp": maxp}
    out = struct.pack(">IHHHH", 0x4F54544F, len(tables), 0, 0, 0)
    at = 12 + 16 * len(tables)
    body = b""
    for tag in sorted(tables):
        data = tables[tag] + b"\x00" * (-len(tables[tag]) % 4)
        out += struct.pack(">4sIII", tag, 0, at + len(body), len(tables[tag]))
        body += data
    return out + body


def points(path):
    return [tuple(round(v, 3) for v in c[-2:]) for contour in path.contours for c in contour]


def _glyphs():
    square = cs(-20, "rmoveto", 0 + 100 - 100, 0, "rmoveto") if False else \
        cs(-100, 100, 50, "rmoveto", 300, "hlineto", 300, "vlineto", -300, "hlineto", "endchar")    # width 600 - 100
    square_alt = cs(100, 50, "rmoveto", 300, 300, -300, "hlineto", "endchar")                     # alternating form
    diamond = cs(50, 0, 20, "hstem", 200, "hmoveto", 150, 150, -150, 150, -150, -150, "rlineto", "endchar")
    ring_rr = cs(400, 200, "rmoveto", 0, 110, -90, 90, -110, 0, -110, 0, -90, -90, 0, -110,
                 0, -110, 90, -90, 110, 0, 110, 0, 90, 90, 0, 110, "rrcurveto", "endchar")
    ring_vh = cs(400, 200, "rmoveto", 110, -90, 90, -110, -110, -90, -90, -110, -110, 90, -90, 110, 110, 90, 90, 110,
                 "vhcurveto", "endchar")
    ring_hint = cs(10, 20, "hstemhm", 30, 40, 50, 60, "hintmask", b"\xe0", 400, 200, "rmoveto", -107 + 0, "callsubr",
                   "endchar")
    ring_sub = cs(110, -90, 90, -110, -110, -90, -90, -110, "vhcurveto", -107, "callgsubr", "return")
    ring_gsub = cs(-110, 90, -90, 110, 110, 90, 90, 110, "vhcurveto", "return")
    mixed = cs(0, "vmoveto", 100, 0, "rlineto", 0, 50, 50, 50, 50, 0, 30, 40, "rcurveline",
               -10, -10, 10, 20, 30, 40, 50, 60, "rlinecurve", "endchar")
    vvhh = cs(0, 0, "rmoveto", 5, 10, 20, 30, 40, "vvcurveto", 7, 10, 20, 30, 40, "hhcurveto", "endchar")
    flexes = cs(0, 0, "rmoveto", 10, 5, 10, 0, 10, -5, 10, -5, 10, 0, 10, 5, 50, "flex",
                10, 20, 5, 10, 10, 20, 10, "hflex", 10, 5, 10, 5, 10, 10, 10, -7, 10, "hflex1",
                10, 5, 10, 0, 10, -5, 10, -5, 10, 0, 13, "flex1", "endchar")
    bad = cs(4, "sqrt", "endchar")
    return [cs("endchar"), square, square_alt, diamond, ring_rr, ring_vh, ring_hint, mixed, vvhh, flexes, bad], \
        [ring_sub], [ring_gsub]


def test_index_and_dict_readers():
    objs, end = read_index(index([b"ab", b"", b"cde"]), 0)
    assert objs == [b"ab", b"", b"cde"] and end == len(index([b"ab", b"", b"cde"]))
    assert read_index(b"\x00\x00rest", 0) == ([], 2)
    d = read_dict(num(-300) + num(1000) + bytes([5]) + int32(70000) + bytes([17]) + b"\x1e\xe2\xa2\x5f" + bytes([12, 7]))
    assert d[5] == [-300, 1000] and d[17] == [70000] and d[1207] == [-2.25]


def test_charstring_operators():
    chars, subrs, gsubrs = _glyphs()
    table = CffTable(build_cff(chars, subrs, gsubrs))
    assert table.num_glyphs == len(chars)
    empty, w0 = table.glyph(0)
    assert not empty.contours and w0 == 500                                  # default width
    sq, w1 = table.glyph(1)
    assert w1 == 500 and points(sq)[:4] == [(100, 50), (400, 50), (400, 350), (100, 350)]      # 600 + (-100)
    assert points(table.glyph(2)[0])[:4] == points(sq)[:4]
    dia, w3 = table.glyph(3)
    assert w3 == 650 and points(dia)[:4] == [(200, 0), (350, 150), (200, 300), (50, 150)]
    a, b, c = (points(table.glyph(g)[0]) for g in (4, 5, 6))
    assert a == b == c and a[0] == (400, 200) and a[1] == (200, 400) and a[2] == (0, 200) and a[4] == (400, 200)
    mixed = points(table.glyph(7)[0])
    assert mixed[:3] == [(0, 0), (100, 0), (200, 100)] and mixed[3] == (230, 140) and mixed[4] == (220, 130)
    assert mixed[5] == (310, 250)
    vvhh = points(table.glyph(8)[0])
    assert vvhh[1] == (5 + 20, 10 + 30 + 40) and vvhh[2] == (25 + 10 + 20 + 40, 80 + 7 + 30)
    fl = points(table.glyph(9)[0])
    assert fl[1:3] == [(30, 0), (60, 0)] and fl[3:5] == [(100, 5), (140, 0)] and fl[5] == (170, 10) and fl[6][1] == 0 and fl[8] == (fl[6][0] + 63, 0)
    with pytest.raises(CffError):
        table.glyph(10)
    assert table.glyph(99)[0].contours == []


def test_open_type_file_with_cff_outlines_renders():
    chars, subrs, gsubrs = _glyphs()
    chars = chars[:10]
    font = im.TrueTypeFont(build_otf(build_cff(chars, subrs, gsubrs), {ord("s"): 1, ord("o"): 4, ord("O"): 6},
                                     [500] * len(chars)))
    assert font.num_glyphs == 10 and font.glyph_index(ord("o")) == 4 and font.units_per_em == 1000
    mask = im.render_text(font, "s", 100, padding=0).float() / 255
    # the square covers (10..40, 5..35) pixels of a 50-wide advance: 900 px of ink
    assert abs(mask.sum().item() - 900) < 1.0
    ring, ring_sub = im.render_text(font, "o", 200, padding=0), im.render_text(font, "O", 200, padding=0)
    assert torch.equal(ring, ring_sub)
    area = (ring.float() / 255).sum().item()
    assert abs(area - 3.14159 * 40 * 40) < 0.02 * 3.14159 * 40 * 40           # radius 200 units = 40 px: a near circle
    with pytest.raises(im.FontError):
        im.TrueTypeFont(b"wOFF" + b"\x00" * 40)


def test_font_collection_faces():
    chars, subrs, gsubrs = _glyphs()
    one = build_otf(build_cff(chars[:4], subrs, gsubrs), {ord("s"): 1}, [500] * 4)
    two = build_otf(build_cff(chars[:6], subrs, gsubrs), {ord("o"): 4}, [700] * 6, upem=2000)

    def shifted(font, by):
        n = struct.unpack(">H", font[4:6])[0]
        out = bytearray(font)
        for i in range(n):
            off = struct.unpack(">I", font[12 + 16 * i + 8: 12 + 16 * i + 12])[0]
            struct.pack_into(">I", out, 12 + 16 * i + 8, off + by)
        return bytes(out)

    header = 12 + 8
    ttc = b"ttcf" + struct.pack(">HHIII", 1, 0, 2, header, header + len(one)) + shifted(one, header) + shifted(two, header + len(one))
    a, b = im.TrueTypeFont(ttc), im.TrueTypeFont(ttc, face=1)
    assert a.num_glyphs == 4 and a.glyph_index(ord("s")) == 1 and a.units_per_em == 1000
    assert b.num_glyphs == 6 and b.glyph_index(ord("o")) == 4 and b.units_per_em == 2000 and b.advance(4) == 700
    assert len(b.glyph_path(4).contours) == 1
    with pytest.raises(im.FontError):
        im.TrueTypeFont(ttc, face=2)
    with pytest.raises(im.FontError):
        im.TrueTypeFont(one, face=1)
