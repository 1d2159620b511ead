"""A small TrueType reader: character map, metrics, glyph outlines (simple and composite ``glyf`` glyphs) and
pair kerning (``kern`` format 0) - enough to lay out a line of text and hand its outline to the coverage rasteriser.

    font = TrueTypeFont(open("font.ttf", "rb").read())
    mask = render_text(font, "Hello", size=32, device="cuda")        # uint8 [H, W] coverage

Outlines come back in font units with y up; ``text_path`` scales to pixels and flips y. Quadratic segments stay
quadratic (the rasteriser flattens them within its tolerance).

Reference: the reference's OpenType engine (src/Idrak.Imaging/Fonts: table readers, glyph outlines, horizontal layout
feeding ``CoverageRasterizer``). CFF outlines, GSUB / GPOS shaping and bidirectional text are not read here.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Optional, Tuple

import torch

from .raster import Path, rasterize


class FontError(ValueError):
    pass


class TrueTypeFont:
    def __init__(self, data: bytes, face: int = 0):
        """``face`` picks a member of a font collection (``ttcf`` container); a single font has face 0 only."""
        self.data = data
        if len(data) < 12:
            raise FontError("not a font file")
        base = 0
        if data[:4] == b"ttcf":
            count = struct.unpack(">I", data[8:12])[0]
            if not 0 <= face < count:
                raise FontError(f"the collection has {count} faces, face {face} was asked for")
            base = struct.unpack(">I", data[12 + 4 * face: 16 + 4 * face])[0]
        elif face != 0:
            raise FontError("a single font file has face 0 only")
        version, n_tables = struct.unpack(">IH", data[base: base + 6])
        if version not in (0x00010000, 0x74727565, 0x4F54544F):       # 1.0, 'true' or 'OTTO' (CFF outlines)
            raise FontError("not a TrueType / OpenType font or collection")
        self.tables: Dict[str, Tuple[int, int]] = {}
        for i in range(n_tables):
            tag, _, off, length = struct.unpack(">4sIII", data[base + 12 + 16 * i: base + 28 + 16 * i])
            self.tables[tag.decode("latin-1")] = (off, length)
        self._cff = None
        outlines = ("CFF ",) if version == 0x4F54544F else ("loca", "glyf")
        for need in ("head", "maxp", "hhea", "hmtx", "cmap") + outlines:
            if need not in self.tables:
                raise FontError(f"the font has no '{need}' table")
        head = self._table("head")
        self.units_per_em = struct.unpack(">H", head[18:20])[0]
        self.long_loca = struct.unpack(">h", head[50:52])[0] == 1
        self.num_glyphs = struct.unpack(">H", self._table("maxp")[4:6])[0]
        hhea = self._table("hhea")
        self.ascender, self.descender, self.line_gap = struct.unpack(">hhh", hhea[4:10])
        self.num_h_metrics = struct.unpack(">H", hhea[34:36])[0]
        self._cmap = self._read_cmap()
        if outlines == ("CFF ",):
            from .cff import CffTable
            self._cff = CffTable(self._table("CFF "))
            self._loca = []
        else:
            self._loca = self._read_loca()
        self._kern = self._read_kern()
        self.gsub = None
        if "GSUB" in self.tables:
            from .gsub import GsubTable
            self.gsub = GsubTable(self._table("GSUB"))
        self._paths: Dict[int, Path] = {}

    def _table(self, tag: str) -> bytes:
        off, length = self.tables[tag]
        return self.data[off: off + length]

    # ------------------------------------------------------------------ tables
    def _read_cmap(self) -> Dict[int, int]:
        t = self._table("cmap")
        n = struct.unpack(">H", t[2:4])[0]
        best, best_rank = None, -1
        for i in range(n):
            plat, enc, off = struct.unpack(">HHI", t[4 + 8 * i: 12 + 8 * i])
            fmt = struct.unpack(">H", t[off: off + 2])[0]
            rank = {(3, 10, 12): 4, (0, 4, 12): 4, (3, 1, 4): 3, (0, 3, 4): 3}.get((plat, enc, fmt), 1 if fmt in (4, 12) else -1)
            if plat in (0, 3) and rank > best_rank:
                best, best_rank = (off, fmt), rank
        if best is None:
            raise FontError("no Unicode character map (format 4 or 12)")
        off, fmt = best
        out: Dict[int, int] = {}
        if fmt == 12:
            n_groups = struct.unpack(">I", t[off + 12: off + 16])[0]
            for g in range(n_groups):
                start, end, gid = struct.unpack(">III", t[off + 16 + 12 * g: off + 28 + 12 * g])
                for c in range(start, end + 1):
                    out[c] = gid + (c - start)
            return out
        seg2 = struct.unpack(">H", t[off + 6: off + 8])[0]
        segs = seg2 // 2
        ends = struct.unpack(f">{segs}H", t[off + 14: off + 14 + seg2])
        base = off + 16 + seg2
        starts = struct.unpack(f">{segs}H", t[base: base + seg2])
        deltas = struct.unpack(f">{segs}h", t[base + seg2: base + 2 * seg2])
        ro_at = base + 2 * seg2
        ranges = struct.unpack(f">{segs}H", t[ro_at: ro_at + seg2])
        for s in range(segs):
            for c in range(starts[s], ends[s] + 1):
                if c == 0xFFFF:
                    continue
                if ranges[s] == 0:
                    gid = (c + deltas[s]) & 0xFFFF
                else:
                    at = ro_at + 2 * s + ranges[s] + 2 * (c - starts[s])
                    gid = struct.unpack(">H", t[at: at + 2])[0]
                    if gid:
                        gid = (gid + deltas[s]) & 0xFFFF
                if gid:
                    out[c] = gid
        return out

    def _read_loca(self) -> List[int]:
        t = self._table("loca")
        n = self.num_glyphs + 1
        if self.long_loca:
            return list(struct.unpack(f">{n}I", t[: 4 * n]))
        return [2 * v for v in struct.unpack(f">{n}H", t[: 2 * n])]

    def _read_kern(self) -> Dict[Tuple[int, int], int]:
        out: Dict[Tuple[int, int], int] = {}
        if "kern" not in self.tables:
            return out
        t = self._table("kern")
        if len(t) < 4 or struct.unpack(">H", t[:2])[0] != 0:
            return out
        n_sub = struct.unpack(">H", t[2:4])[0]
        at = 4
        for _ in range(n_sub):
            _, length, coverage = struct.unpack(">HHH", t[at: at + 6])
            if coverage >> 8 == 0 and coverage & 1:          # format 0, horizontal
                pairs = struct.unpack(">H", t[at + 6: at + 8])[0]
                for i in range(pairs):
                    l, r, v = struct.unpack(">HHh", t[at + 14 + 6 * i: at + 20 + 6 * i])
                    out[(l, r)] = v
            at += length
        return out

    # ------------------------------------------------------------------ queries
    def glyph_index(self, codepoint: int) -> int:
        return self._cmap.get(codepoint, 0)

    def advance(self, gid: int) -> int:
        t = self._table("hmtx")
        i = min(gid, self.num_h_metrics - 1)
        return struct.unpack(">H", t[4 * i: 4 * i + 2])[0]

    def kerning(self, left: int, right: int) -> int:
        return self._kern.get((left, right), 0)

    def glyph_path(self, gid: int, _depth: int = 0) -> Path:
        """The glyph's outline in font units, y up."""
        if gid in self._paths:
            return self._paths[gid]
        path = Path()
        if self._cff is not None:
            path = self._cff.glyph(gid)[0]
        elif 0 <= gid < self.num_glyphs and self._loca[gid + 1] > self._loca[gid] and _depth < 8:
            g = self._table("glyf")[self._loca[gid]: self._loca[gid + 1]]
            n_contours = struct.unpack(">h", g[:2])[0]
            if n_contours >= 0:
                self._simple(g, n_contours, path)
            else:
                self._composite(g, path, _depth)
        self._paths[gid] = path
        return path

    def _simple(self, g: bytes, n_contours: int, path: Path) -> None:
        ends = struct.unpack(f">{n_contours}H", g[10: 10 + 2 * n_contours])
        n_points = ends[-1] + 1 if n_contours else 0
        at = 10 + 2 * n_contours
        n_instr = struct.unpack(">H", g[at: at + 2])[0]
        at += 2 + n_instr
        flags: List[int] = []
        while len(flags) < n_points:
            f = g[at]
            at += 1
            flags.append(f)
            if f & 8:
                rep = g[at]
                at += 1
                flags.extend([f] * rep)
        flags = flags[:n_points]

        def coords(short_bit: int, same_bit: int) -> List[int]:
            nonlocal at
            out, v = [], 0
            for f in flags:
                if f & short_bit:
                    d = g[at]
                    at += 1
                    v += d if f & same_bit else -d
                elif not f & same_bit:
                    v += struct.unpack(">h", g[at: at + 2])[0]
                    at += 2
                out.append(v)
            return out

        xs = coords(2, 16)
        ys = coords(4, 32)
        start = 0
        for end in ends:
            pts = [(xs[i], ys[i], bool(flags[i] & 1)) for i in range(start, end + 1)]
            start = end + 1
            _contour_to_path(pts, path)

    def _composite(self, g: bytes, path: Path, depth: int) -> None:
        at = 10
        while True:
            flags, gid = struct.unpack(">HH", g[at: at + 4])
            at += 4
            if flags & 1:
                a1, a2 = struct.unpack(">hh", g[at: at + 4])
                at += 4
            else:
                a1, a2 = struct.unpack(">bb", g[at: at + 2])
                at += 2
            a = d = 1.0
            b = c = 0.0
            if flags & 8:
                a = d = struct.unpack(">h", g[at: at + 2])[0] / 16384.0
                at += 2
            elif flags & 0x40:
                a, d = (v / 16384.0 for v in struct.unpack(">hh", g[at: at + 4]))
                at += 4
            elif flags & 0x80:
                a, b, c, d = (v / 16384.0 for v in struct.unpack(">hhhh", g[at: at + 8]))
                at += 8
            dx, dy = (a1, a2) if flags & 2 else (0, 0)      # point-matching offsets are not resolved
            child = self.glyph_path(gid, depth + 1)
            for contour in child.contours:
                new = []
                for cmd in contour:
                    p = cmd[1:]
                    new.append((cmd[0],) + tuple(v for i in range(0, len(p), 2)
                                                 for v in (a * p[i] + c * p[i + 1] + dx, b * p[i] + d * p[i + 1] + dy)))
                path.contours.append(new)
            if not flags & 0x20:
                break

    # ------------------------------------------------------------------ layout
    def layout(self, text: str, size: float, kerning: bool = True, shape: bool = True) -> List[Tuple[int, float]]:
        """(glyph id, pen x in pixels) per character, left to right on one line. A line with right-to-left
        characters is shaped (Arabic contextual forms) and put into drawing order first (``imaging/shaping.py``);
        a presentation form the font has no glyph for falls back to its base letter."""
        scale = size / self.units_per_em
        pen, prev, out = 0.0, None, []
        glyphs: List[int] = []
        rtl = shape and any("\u0590" <= ch <= "\u08ff" or "\ufb1d" <= ch <= "\ufefc" for ch in text)
        if rtl and self.gsub is not None and self.gsub.joins:
            glyphs = self._shape_with_gsub(text)
        else:
            if rtl:
                from .shaping import layout_line
                text = layout_line(text)
            for ch in text:
                gid = self.glyph_index(ord(ch))
                if gid == 0 and "\ufe70" <= ch <= "\ufefc":
                    import unicodedata
                    base = [int(b, 16) for b in unicodedata.decomposition(ch).split()[1:]]
                    # a ligature the font lacks: its letters, last first (the line is already in drawing order)
                    glyphs += [self.glyph_index(b) for b in reversed(base)] or [0]
                else:
                    glyphs.append(gid)
        for gid in glyphs:
            if kerning and prev is not None:
                pen += self.kerning(prev, gid) * scale
            out.append((gid, pen))
            pen += self.advance(gid) * scale
            prev = gid
        return out

    def _shape_with_gsub(self, text: str) -> List[int]:
        """Glyphs of a line with right-to-left text in drawing order, the positional forms and the required / standard
        ligatures taken from the font's own substitution table."""
        from .shaping import _MIRROR, arabic_forms, visual_indices
        tags = {"isolated": "isol", "initial": "init", "medial": "medi", "final": "fina"}
        per_char: List[List[int]] = []
        for ch, form in arabic_forms(text):
            gid = self.glyph_index(ord(ch))
            per_char.append(list(self.gsub.single(tags[form]).get(gid, (gid,))) if form else [gid])
        # ligatures over the logical sequence: the first character keeps the ligature, the others lose their glyphs
        for tag in ("rlig", "liga"):
            rules = self.gsub.ligatures(tag)
            i = 0
            while rules and i < len(per_char):
                if len(per_char[i]) == 1:
                    for rest, lig in rules.get(per_char[i][0], []):
                        follow = per_char[i + 1: i + 1 + len(rest)]
                        if len(follow) == len(rest) and all(len(f) == 1 and f[0] == r for f, r in zip(follow, rest)) \
                                and (tag == "rlig" or all("\u0590" <= text[k] <= "\u08ff" for k in range(i, i + 1 + len(rest)))):
                            per_char[i] = [lig]
                            for k in range(i + 1, i + 1 + len(rest)):
                                per_char[k] = []
                            break
                i += 1
        out: List[int] = []
        for i, mirrored in visual_indices(text):
            if mirrored:
                out.append(self.glyph_index(ord(_MIRROR[text[i]])))
            else:
                from .shaping import _direction
                out += reversed(per_char[i]) if _direction(text[i]) == "R" else per_char[i]
        return out

    def measure(self, text: str, size: float) -> Tuple[float, float, float]:
        """(advance width, ascent, descent) of the line in pixels (descent positive downwards)."""
        scale = size / self.units_per_em
        placed = self.layout(text, size)
        width = placed[-1][1] + self.advance(placed[-1][0]) * scale if placed else 0.0
        return width, self.ascender * scale, -self.descender * scale

    def text_path(self, text: str, size: float, x: float = 0.0, baseline: float = 0.0, shear: float = 0.0) -> Path:
        """The line's outline in pixels (y down) with its origin at (x, baseline)."""
        scale = size / self.units_per_em
        out = Path()
        for gid, pen in self.layout(text, size):
            out.contours += self.glyph_path(gid).transformed(scale, -scale, x + pen, baseline, shear=-shear * scale).contours
        return out


def _contour_to_path(pts: List[Tuple[int, int, bool]], path: Path) -> None:
    """TrueType points (on / off curve, implied on-curve midpoints between two off-curve points) -> move / line / quad."""
    if not pts:
        return
    n = len(pts)
    # start at an on-curve point; if there is none, at the midpoint of the first two off-curve points
    first = next((i for i, p in enumerate(pts) if p[2]), None)
    if first is None:
        sx, sy = (pts[0][0] + pts[1 % n][0]) / 2.0, (pts[0][1] + pts[1 % n][1]) / 2.0
        order = [pts[(1 + i) % n] for i in range(n)]
    else:
        sx, sy = float(pts[first][0]), float(pts[first][1])
        order = [pts[(first + 1 + i) % n] for i in range(n)]       # ends with the start point itself
    path.move_to(sx, sy)
    ctrl: Optional[Tuple[float, float]] = None
    for x, y, on in order:
        if on:
            if ctrl is None:
                path.line_to(x, y)
            else:
                path.quad_to(ctrl[0], ctrl[1], x, y)
                ctrl = None
        else:
            if ctrl is not None:
                mx, my = (ctrl[0] + x) / 2.0, (ctrl[1] + y) / 2.0
                path.quad_to(ctrl[0], ctrl[1], mx, my)
            ctrl = (float(x), float(y))
    if ctrl is not None:
        path.quad_to(ctrl[0], ctrl[1], sx, sy)


def render_text(font: TrueTypeFont, text: str, size: float, padding: int = 2, device: Optional[str] = None,
                dtype: torch.dtype = torch.uint8, shear: float = 0.0) -> torch.Tensor:
    """Coverage mask ``[H, W]`` of one line of text: H = ascent + descent + 2 padding, W = advance + 2 padding."""
    import math
    width, ascent, descent = font.measure(text, size)
    W = max(int(math.ceil(width + abs(shear) * (ascent + descent))) + 2 * padding, 1)
    H = max(int(math.ceil(ascent + descent)) + 2 * padding, 1)
    path = font.text_path(text, size, x=padding + (abs(shear) * descent if shear else 0.0), baseline=padding + ascent, shear=shear)
    return rasterize([path], W, H, device=device, dtype=dtype)[0]
