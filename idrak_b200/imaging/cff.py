"""Compact Font Format outlines: the ``CFF`` table of an OpenType font (``OTTO`` flavour) and its Type 2 charstrings.

``CffTable`` reads the header, the INDEX structures (names, top dictionaries, strings, global subroutines, charstrings),
the top and private dictionaries (CID-keyed fonts: one private dictionary per font dictionary, chosen per glyph through
FDSelect formats 0 and 3) and interprets a glyph's charstring into a ``Path`` of lines and cubic curves in font units:
every move / line / curve operator (``rmoveto`` … ``hvcurveto``, ``rcurveline``, ``rlinecurve``), the four flex
operators, stem hints and hint masks (counted so that the mask bytes are skipped; hints themselves are not applied -
the rasteriser works at exact coverage), local and global subroutines with the size-dependent bias, and the optional
leading width. Arithmetic and storage operators (``12 x`` other than flex) are rejected by name.

Reference: the CFF reader of the reference's font stack (src/Idrak.Imaging/Text).
"""
from __future__ import annotations

import struct
from typing import Dict, List, Optional, Tuple

from .raster import Path


class CffError(ValueError):
    pass


def read_index(data: bytes, at: int) -> Tuple[List[bytes], int]:
    """An INDEX at ``at`` -> (its objects, the offset just past it)."""
    count = struct.unpack(">H", data[at: at + 2])[0]
    if count == 0:
        return [], at + 2
    size = data[at + 2]
    if not 1 <= size <= 4:
        raise CffError("bad INDEX offset size")
    base = at + 3 + (count + 1) * size - 1
    offs = [int.from_bytes(data[at + 3 + i * size: at + 3 + (i + 1) * size], "big") for i in range(count + 1)]
    return [data[base + offs[i]: base + offs[i + 1]] for i in range(count)], base + offs[-1]


def read_dict(data: bytes) -> Dict[int, List[float]]:
    """A DICT -> {operator: operands}; two-byte operators are 1200 + the second byte."""
    out: Dict[int, List[float]] = {}
    stack: List[float] = []
    i, n = 0, len(data)
    while i < n:
        b = data[i]
        if b <= 21:
            op = b
            i += 1
            if b == 12:
                op = 1200 + data[i]
                i += 1
            out[op] = stack
            stack = []
        elif b == 28:
            stack.append(struct.unpack(">h", data[i + 1: i + 3])[0]); i += 3
        elif b == 29:
            stack.append(struct.unpack(">i", data[i + 1: i + 5])[0]); i += 5
        elif b == 30:                                           # real number: packed nibbles
            text, i = "", i + 1
            done = False
            while not done:
                for nib in (data[i] >> 4, data[i] & 15):
                    if nib == 15:
                        done = True
                        break
                    text += "0123456789.EE?-"[nib] if nib != 12 else "E-"
                i += 1
            stack.append(float(text))
        elif 32 <= b <= 246:
            stack.append(b - 139); i += 1
        elif 247 <= b <= 250:
            stack.append((b - 247) * 256 + data[i + 1] + 108); i += 2
        elif 251 <= b <= 254:
            stack.append(-(b - 251) * 256 - data[i + 1] - 108); i += 2
        else:
            raise CffError(f"bad DICT byte {b}")
    return out


def _bias(count: int) -> int:
    return 107 if count < 1240 else 1131 if count < 33900 else 32768


class CffTable:
    def __init__(self, data: bytes):
        self.data = data
        if len(data) < 4 or data[0] != 1:
            raise CffError("only CFF version 1 is read")
        at = data[2]
        _, at = read_index(data, at)                            # names
        tops, at = read_index(data, at)
        _, at = read_index(data, at)                            # strings
        self.global_subrs, _ = read_index(data, at)
        if not tops:
            raise CffError("no top dictionary")
        top = read_dict(tops[0])
        if 17 not in top:
            raise CffError("no charstrings")
        self.charstrings, _ = read_index(data, int(top[17][0]))
        self.num_glyphs = len(self.charstrings)
        self.matrix = top.get(1207, [0.001, 0, 0, 0.001, 0, 0])
        self._privates: List[Tuple[List[bytes], float, float]] = []
        self._fd_select: Optional[List[int]] = None
        if 1230 in top:                                         # CID-keyed: font dictionaries + a selector per glyph
            fds, _ = read_index(data, int(top[1236][0]))
            for fd in fds:
                self._privates.append(self._private(read_dict(fd)))
            self._fd_select = self._read_fd_select(int(top[1237][0]))
        else:
            self._privates.append(self._private(top))

    def _private(self, d: Dict[int, List[float]]) -> Tuple[List[bytes], float, float]:
        if 18 not in d:
            return [], 0.0, 0.0
        size, off = int(d[18][0]), int(d[18][1])
        p = read_dict(self.data[off: off + size])
        subrs: List[bytes] = []
        if 19 in p:
            subrs, _ = read_index(self.data, off + int(p[19][0]))
        return subrs, float(p.get(20, [0])[0]), float(p.get(21, [0])[0])

    def _read_fd_select(self, at: int) -> List[int]:
        fmt = self.data[at]
        if fmt == 0:
            return list(self.data[at + 1: at + 1 + self.num_glyphs])
        if fmt == 3:
            n = struct.unpack(">H", self.data[at + 1: at + 3])[0]
            out = [0] * self.num_glyphs
            for i in range(n):
                first, fd = struct.unpack(">HB", self.data[at + 3 + 3 * i: at + 6 + 3 * i])
                nxt = struct.unpack(">H", self.data[at + 6 + 3 * i: at + 8 + 3 * i])[0]
                for g in range(first, min(nxt, self.num_glyphs)):
                    out[g] = fd
            return out
        raise CffError(f"FDSelect format {fmt} is not read")

    # -------------------------------------------------------------------------------------------------- charstrings
    def glyph(self, gid: int) -> Tuple[Path, Optional[float]]:
        """(outline in font units with y up, advance width from the charstring or None when it has none)."""
        path = Path()
        if not 0 <= gid < self.num_glyphs:
            return path, None
        subrs, default_w, nominal_w = self._privates[self._fd_select[gid] if self._fd_select else 0]
        st = _Run(path, subrs, self.global_subrs, nominal_w)
        st.run(self.charstrings[gid], 0)
        if st.open:
            path.close()
        return path, (st.width if st.width is not None else default_w)


class _Run:
    def __init__(self, path: Path, subrs: List[bytes], gsubrs: List[bytes], nominal: float):
        self.path, self.subrs, self.gsubrs, self.nominal = path, subrs, gsubrs, nominal
        self.stack: List[float] = []
        self.x = self.y = 0.0
        self.stems = 0
        self.width: Optional[float] = None
        self.seen_width = False
        self.open = False
        self.done = False

    # the first stack-clearing operator may carry the width in front of its own operands
    def _take_width(self, expected: int, parity: bool = False) -> None:
        if self.seen_width:
            return
        self.seen_width = True
        extra = (len(self.stack) % 2 == 1) if parity else len(self.stack) > expected
        if extra:
            self.width = self.nominal + self.stack.pop(0)

    def _move(self, dx: float, dy: float) -> None:
        if self.open:
            self.path.close()
        self.x += dx; self.y += dy
        self.path.move_to(self.x, self.y)
        self.open = True

    def _line(self, dx: float, dy: float) -> None:
        self.x += dx; self.y += dy
        self.path.line_to(self.x, self.y)

    def _curve(self, a: float, b: float, c: float, d: float, e: float, f: float) -> None:
        x1, y1 = self.x + a, self.y + b
        x2, y2 = x1 + c, y1 + d
        self.x, self.y = x2 + e, y2 + f
        self.path.cubic_to(x1, y1, x2, y2, self.x, self.y)

    def run(self, code: bytes, depth: int) -> None:
        if depth > 10:
            raise CffError("subroutines nested too deeply")
        s = self.stack
        i, n = 0, len(code)
        while i < n and not self.done:
            b = code[i]
            if b >= 32 or b == 28:
                if b == 28:
                    s.append(struct.unpack(">h", code[i + 1: i + 3])[0]); i += 3
                elif b <= 246:
                    s.append(b - 139); i += 1
                elif b <= 250:
                    s.append((b - 247) * 256 + code[i + 1] + 108); i += 2
                elif b <= 254:
                    s.append(-(b - 251) * 256 - code[i + 1] - 108); i += 2
                else:
                    s.append(struct.unpack(">i", code[i + 1: i + 5])[0] / 65536.0); i += 5
                continue
            i += 1
            if b in (1, 3, 18, 23):                              # stems
                self._take_width(0, parity=True)
                self.stems += len(s) // 2
                s.clear()
            elif b in (19, 20):                                  # hint / counter mask (implied vstem before the first)
                self._take_width(0, parity=True)
                self.stems += len(s) // 2
                s.clear()
                i += (self.stems + 7) // 8
            elif b == 21:
                self._take_width(2); self._move(s[0], s[1]); s.clear()
            elif b == 22:
                self._take_width(1); self._move(s[0], 0); s.clear()
            elif b == 4:
                self._take_width(1); self._move(0, s[0]); s.clear()
            elif b == 5:
                for k in range(0, len(s) - 1, 2):
                    self._line(s[k], s[k + 1])
                s.clear()
            elif b in (6, 7):                                    # alternating horizontal / vertical lines
                horizontal = b == 6
                for v in s:
                    self._line(v, 0) if horizontal else self._line(0, v)
                    horizontal = not horizontal
                s.clear()
            elif b == 8:
                for k in range(0, len(s) - 5, 6):
                    self._curve(*s[k: k + 6])
                s.clear()
            elif b == 24:                                        # curves then a line
                k = 0
                while k + 6 <= len(s) - 2:
                    self._curve(*s[k: k + 6]); k += 6
                self._line(s[k], s[k + 1]); s.clear()
            elif b == 25:                                        # lines then a curve
                k = 0
                while k + 2 <= len(s) - 6:
                    self._line(s[k], s[k + 1]); k += 2
                self._curve(*s[k: k + 6]); s.clear()
            elif b == 26:                                        # vvcurveto
                k, dx = 0, 0.0
                if len(s) % 4 == 1:
                    dx, k = s[0], 1
                while k + 4 <= len(s):
                    self._curve(dx, s[k], s[k + 1], s[k + 2], 0, s[k + 3]); dx = 0.0; k += 4
                s.clear()
            elif b == 27:                                        # hhcurveto
                k, dy = 0, 0.0
                if len(s) % 4 == 1:
                    dy, k = s[0], 1
                while k + 4 <= len(s):
                    self._curve(s[k], dy, s[k + 1], s[k + 2], s[k + 3], 0); dy = 0.0; k += 4
                s.clear()
            elif b in (30, 31):                                  # vhcurveto / hvcurveto: tangents alternate
                horizontal = b == 31
                k = 0
                while k + 4 <= len(s):
                    last = s[k + 4] if len(s) - k == 5 else 0.0
                    if horizontal:
                        self._curve(s[k], 0, s[k + 1], s[k + 2], last, s[k + 3])
                    else:
                        self._curve(0, s[k], s[k + 1], s[k + 2], s[k + 3], last)
                    horizontal = not horizontal
                    k += 4
                s.clear()
            elif b == 10 or b == 29:
                table = self.subrs if b == 10 else self.gsubrs
                idx = int(s.pop()) + _bias(len(table))
                if not 0 <= idx < len(table):
                    raise CffError("subroutine index out of range")
                self.run(table[idx], depth + 1)
            elif b == 11:
                return
            elif b == 14:
                self._take_width(4 if len(s) >= 4 else 0)
                self.done = True
            elif b == 12:
                op = code[i]; i += 1
                if op == 35:                                     # flex: two curves, the 13th operand is the flex depth
                    self._curve(*s[0:6]); self._curve(*s[6:12])
                elif op == 34:                                   # hflex
                    self._curve(s[0], 0, s[1], s[2], s[3], 0); self._curve(s[4], 0, s[5], -s[2], s[6], 0)
                elif op == 36:                                   # hflex1
                    self._curve(s[0], s[1], s[2], s[3], s[4], 0)
                    self._curve(s[5], 0, s[6], s[7], s[8], -(s[1] + s[3] + s[7]))
                elif op == 37:                                   # flex1: the last operand closes the larger extent
                    x0, y0 = self.x, self.y
                    dx = s[0] + s[2] + s[4] + s[6] + s[8]
                    dy = s[1] + s[3] + s[5] + s[7] + s[9]
                    self._curve(*s[0:6])
                    if abs(dx) > abs(dy):
                        self._curve(s[6], s[7], s[8], s[9], s[10], y0 - (self.y + s[7] + s[9]))
                    else:
                        self._curve(s[6], s[7], s[8], s[9], x0 - (self.x + s[6] + s[8]), s[10])
                else:
                    raise CffError(f"charstring operator 12 {op} is not supported")
                s.clear()
            else:
                raise CffError(f"charstring operator {b} is not supported")
