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


def build_otf(cff, cmap, advances, upem=1000, extra=None):
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
    tables.update(extra or {})
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


def build_gsub():
    """Features init / medi / fina (single substitutions, both formats, one behind an extension lookup), isol as a
    multiple substitution, rlig with one ligature. Glyphs: 1 beh, 2 lam, 3 alef; 4-6 beh init / medi / fina;
    7-9 lam init / medi / fina; 10 alef fina; 11 lam-alef (from lam.init + alef.fina), 12 lam-alef joined
    (lam.medi + alef.fina); 13 + 14 = beh isolated as a base and a dot."""
    H = lambda *v: struct.pack(f">{len(v)}H", *v)
    cov = lambda glyphs: H(1, len(glyphs), *glyphs)
    single2 = lambda pairs: H(2, 6 + 2 * len(pairs), len(pairs), *[b for _, b in pairs]) + cov([a for a, _ in pairs])
    init = single2([(1, 4), (2, 7)])
    medi = single2([(1, 5), (2, 8)])
    fina_sub = H(1, 6) + struct.pack(">h", 5) + cov([1])                          # beh 1 -> 6 by delta
    fina_sub2 = single2([(2, 9), (3, 10)])
    # multiple substitution format 1: format, coverageOffset, sequenceCount, sequenceOffsets[], then the tables
    seq = H(2, 13, 14)
    isol = H(1, 8 + len(seq), 1, 8) + seq + cov([1])
    lig = lambda glyph, *rest: H(glyph, 1 + len(rest), *rest)
    set7 = H(1, 4) + lig(11, 10)
    set8 = H(1, 4) + lig(12, 10)
    liga = H(1, 10 + len(set7) + len(set8), 2, 10, 10 + len(set7)) + set7 + set8 + cov([7, 8])

    def lookup(kind, *subs):
        head = H(kind, 0, len(subs))
        offs, at = [], 6 + 2 * len(subs)
        for sub in subs:
            offs.append(at)
            at += len(sub)
        return head + H(*offs) + b"".join(subs)

    ext = H(1, 1) + struct.pack(">I", 8)                                         # extension -> type 1 right behind it
    lookups = [lookup(1, init), lookup(1, medi), lookup(1, fina_sub, fina_sub2), lookup(2, isol), lookup(4, liga),
               lookup(7, ext + single2([(1, 6)]))]
    offs, at = [], 2 + 2 * len(lookups)
    for l in lookups:
        offs.append(at)
        at += len(l)
    lookup_list = H(len(lookups), *offs) + b"".join(lookups)
    feats = [(b"fina", [2, 5]), (b"init", [0]), (b"isol", [3]), (b"medi", [1]), (b"rlig", [4])]
    records, tables, at = b"", b"", 2 + 6 * len(feats)
    for tag, idx in feats:
        records += tag + H(at)
        table = H(0, len(idx), *idx)
        tables += table
        at += len(table)
    feature_list = H(len(feats)) + records + tables
    script_list = H(0)
    return H(1, 0, 10, 10 + len(script_list), 10 + len(script_list) + len(feature_list)) + script_list + feature_list + lookup_list


def test_gsub_forms_and_ligatures_drive_the_line_layout():
    from idrak_b200.imaging.gsub import GsubTable
    g = GsubTable(build_gsub())
    assert g.joins and sorted(g.features) == ["fina", "init", "isol", "medi", "rlig"]
    assert g.single("init") == {1: (4,), 2: (7,)} and g.single("medi") == {1: (5,), 2: (8,)}
    assert g.single("fina") == {1: (6,), 2: (9,), 3: (10,)} and g.single("isol") == {1: (13, 14)}
    assert g.ligatures("rlig") == {7: [((10,), 11)], 8: [((10,), 12)]} and g.single("kern") == {}
    chars, subrs, gsubrs = _glyphs()
    glyphs = [chars[0]] + [chars[1]] * 14
    font = im.TrueTypeFont(build_otf(build_cff(glyphs, subrs, gsubrs), {0x628: 1, 0x644: 2, 0x627: 3, ord("a"): 1},
                                     [500] * 15, extra={b"GSUB": build_gsub()}))
    ids = lambda text: [gid for gid, _ in font.layout(text, 10)]
    assert ids("ببب") == [6, 5, 4]                       # drawing order: final, medial, initial
    assert ids("ب") == [14, 13]                           # isolated: base and dot, reversed with the run
    assert ids("بلا") == [12, 4]                          # beh.init + (lam.medi + alef.fina -> joined ligature)
    assert ids("لا") == [11]
    assert ids("a بب") == [1, 0, 6, 4]                    # a left-to-right line: the Arabic run reversed inside it
    assert ids("ab") == [1, 0]
