"""Glyph substitution table (``GSUB``) of an OpenType font, as far as joining scripts need it: the feature list, single
and multiple substitutions (lookup types 1 and 2: the ``isol`` / ``init`` / ``medi`` / ``fina`` forms) and ligatures (type 4:
``rlig`` / ``liga``, the lam-alef family), with coverage formats 1 and 2 and extension lookups (type 7). Script and
language systems are not distinguished: a feature tag stands for the union of its lookups over all of them. Contextual
lookups (types 5, 6, 8) are skipped.

Reference: the GSUB part of the reference's text shaping (src/Idrak.Imaging/Text).
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple


def _u16(t: bytes, at: int) -> int:
    return struct.unpack(">H", t[at: at + 2])[0]


def _coverage(t: bytes, at: int) -> List[int]:
    """Glyph ids in coverage order."""
    fmt, n = _u16(t, at), _u16(t, at + 2)
    if fmt == 1:
        return list(struct.unpack(f">{n}H", t[at + 4: at + 4 + 2 * n]))
    out: List[int] = []
    if fmt == 2:
        for i in range(n):
            start, end, _ = struct.unpack(">HHH", t[at + 4 + 6 * i: at + 10 + 6 * i])
            out.extend(range(start, end + 1))
    return out


class GsubTable:
    def __init__(self, data: bytes):
        self.t = data
        self.features: Dict[str, List[int]] = {}
        if len(data) < 10 or _u16(data, 0) != 1:
            return
        feat_at, self._lookups_at = _u16(data, 6), _u16(data, 8)
        for i in range(_u16(data, feat_at)):
            tag = data[feat_at + 2 + 6 * i: feat_at + 6 + 6 * i].decode("latin-1")
            f = feat_at + _u16(data, feat_at + 6 + 6 * i)
            lookups = [_u16(data, f + 4 + 2 * k) for k in range(_u16(data, f + 2))]
            have = self.features.setdefault(tag, [])
            have += [l for l in lookups if l not in have]
        self._single: Dict[str, Dict[int, Tuple[int, ...]]] = {}
        self._liga: Dict[str, Dict[int, List[Tuple[Tuple[int, ...], int]]]] = {}

    def _subtables(self, lookup: int) -> List[Tuple[int, int]]:
        """(type, absolute offset) of a lookup's subtables, extension lookups resolved."""
        t, base = self.t, self._lookups_at
        if lookup >= _u16(t, base):
            return []
        at = base + _u16(t, base + 2 + 2 * lookup)
        kind, n = _u16(t, at), _u16(t, at + 4)
        out = []
        for k in range(n):
            sub = at + _u16(t, at + 6 + 2 * k)
            if kind == 7 and _u16(t, sub) == 1:
                out.append((_u16(t, sub + 2), sub + struct.unpack(">I", t[sub + 4: sub + 8])[0]))
            else:
                out.append((kind, sub))
        return out

    def single(self, tag: str) -> Dict[int, Tuple[int, ...]]:
        """glyph -> its replacement glyphs under the feature ``tag`` (empty when the font has none): one glyph from a
        single substitution (type 1), one or several from a multiple substitution (type 2, e.g. a base shape and its
        dots as separate glyphs)."""
        if tag in self._single:
            return self._single[tag]
        out: Dict[int, Tuple[int, ...]] = {}
        t = self.t
        for lookup in self.features.get(tag, []):
            for kind, at in self._subtables(lookup):
                if kind not in (1, 2):
                    continue
                fmt, cov = _u16(t, at), _coverage(t, at + _u16(t, at + 2))
                if kind == 1 and fmt == 1:
                    delta = struct.unpack(">h", t[at + 4: at + 6])[0]
                    for g in cov:
                        out.setdefault(g, ((g + delta) & 0xFFFF,))
                elif kind == 1 and fmt == 2:
                    for i, g in enumerate(cov[: _u16(t, at + 4)]):
                        out.setdefault(g, (_u16(t, at + 6 + 2 * i),))
                elif kind == 2 and fmt == 1:
                    for i, g in enumerate(cov[: _u16(t, at + 4)]):
                        seq = at + _u16(t, at + 6 + 2 * i)
                        n = _u16(t, seq)
                        out.setdefault(g, tuple(struct.unpack(f">{n}H", t[seq + 2: seq + 2 + 2 * n])))
        self._single[tag] = out
        return out

    def ligatures(self, tag: str) -> Dict[int, List[Tuple[Tuple[int, ...], int]]]:
        """first glyph -> [(the following components, ligature glyph)], longest first."""
        if tag in self._liga:
            return self._liga[tag]
        out: Dict[int, List[Tuple[Tuple[int, ...], int]]] = {}
        t = self.t
        for lookup in self.features.get(tag, []):
            for kind, at in self._subtables(lookup):
                if kind != 4 or _u16(t, at) != 1:
                    continue
                cov = _coverage(t, at + _u16(t, at + 2))
                for i, first in enumerate(cov[: _u16(t, at + 4)]):
                    lig_set = at + _u16(t, at + 6 + 2 * i)
                    for k in range(_u16(t, lig_set)):
                        lig = lig_set + _u16(t, lig_set + 2 + 2 * k)
                        glyph, comps = _u16(t, lig), _u16(t, lig + 2)
                        rest = tuple(struct.unpack(f">{comps - 1}H", t[lig + 4: lig + 4 + 2 * (comps - 1)])) if comps > 1 else ()
                        out.setdefault(first, []).append((rest, glyph))
        for rules in out.values():
            rules.sort(key=lambda r: -len(r[0]))
        self._liga[tag] = out
        return out

    @property
    def joins(self) -> bool:
        """Does the font carry positional forms (any of ``init`` / ``medi`` / ``fina``)?"""
        return any(self.features.get(tag) for tag in ("init", "medi", "fina"))
