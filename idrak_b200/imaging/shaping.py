"""Text shaping for right-to-left scripts before rasterisation: Arabic contextual forms with the lam-alef ligatures,
and a visual reordering of mixed-direction lines.

``shape_arabic`` turns a string in logical order into presentation forms (isolated / initial / medial / final),
chosen from the joining behaviour of each letter's neighbours; combining marks are transparent. The form tables are
not written out here: they are read from the Unicode character database (every code point of the Arabic Presentation
Forms-B block carries its base letter and form in its compatibility decomposition), so they are as complete as the
interpreter's ``unicodedata``.

``visual_order`` is a small bidirectional algorithm: the base direction comes from the first strong character, the
line is cut into directional runs (letters are strong, European digits keep left-to-right order inside a right-to-left
run, neutrals between two runs of one direction join them, otherwise they take the base direction), right-to-left
runs are reversed and, in a right-to-left line, the runs themselves are laid out from the right; mirrored punctuation
(brackets) is swapped in reversed runs. ``layout_line`` does both and is what the text rasteriser needs: code points in
left-to-right drawing order.

Reference: the shaping and bidirectional steps of the reference's text rendering (src/Idrak.Imaging/Text).
"""
from __future__ import annotations

import unicodedata
from functools import lru_cache
from typing import Dict, List, Tuple

ISOLATED, FINAL, INITIAL, MEDIAL = "isolated", "final", "initial", "medial"
_MIRROR = {"(": ")", ")": "(", "[": "]", "]": "[", "{": "}", "}": "{", "<": ">", ">": "<", "«": "»", "»": "«"}


@lru_cache(maxsize=1)
def _tables() -> Tuple[Dict[str, Dict[str, str]], Dict[Tuple[str, str], Dict[str, str]]]:
    """(letter -> {form: presentation character}, (lam, alef) -> {form: ligature})."""
    letters: Dict[str, Dict[str, str]] = {}
    ligatures: Dict[Tuple[str, str], Dict[str, str]] = {}
    for cp in range(0xFE70, 0xFEFD):
        d = unicodedata.decomposition(chr(cp))
        if not d.startswith("<"):
            continue
        tag, *points = d.split()
        form = tag.strip("<>")
        if form not in (ISOLATED, FINAL, INITIAL, MEDIAL):
            continue
        chars = [chr(int(p, 16)) for p in points]
        if len(chars) == 1:
            letters.setdefault(chars[0], {})[form] = chr(cp)
        elif len(chars) == 2 and chars[0] == "ل":                  # lam + an alef
            ligatures.setdefault((chars[0], chars[1]), {})[form] = chr(cp)
    return letters, ligatures


def _is_mark(ch: str) -> bool:
    return unicodedata.category(ch) in ("Mn", "Me", "Cf") and ch != "‍"


def _joins_left(ch: str) -> bool:
    """Can ``ch`` connect to the letter that follows it (on its left in a right-to-left line)?"""
    if ch == "‍" or ch == "ـ":                                # zero-width joiner, tatweel
        return True
    forms = _tables()[0].get(ch)
    return bool(forms) and INITIAL in forms


def _joins_right(ch: str) -> bool:
    """Can ``ch`` connect to the letter before it?"""
    if ch == "‍" or ch == "ـ":
        return True
    forms = _tables()[0].get(ch)
    return bool(forms) and FINAL in forms


def arabic_forms(text: str) -> List[Tuple[str, str]]:
    """Per character of ``text`` (logical order): (the character, its joining form or "" for anything that has none)."""
    letters, _ = _tables()
    chars = list(text)
    n = len(chars)

    def neighbour(i: int, step: int) -> str:
        j = i + step
        while 0 <= j < n and _is_mark(chars[j]):
            j += step
        return chars[j] if 0 <= j < n else ""

    out: List[Tuple[str, str]] = []
    for i, ch in enumerate(chars):
        forms = letters.get(ch)
        if not forms:
            out.append((ch, ""))
            continue
        prev, nxt = neighbour(i, -1), neighbour(i, +1)
        before = bool(prev) and _joins_left(prev) and FINAL in forms
        after = bool(nxt) and _joins_right(nxt) and INITIAL in forms
        out.append((ch, MEDIAL if before and after and MEDIAL in forms else INITIAL if after else FINAL if before else ISOLATED))
    return out


def shape_arabic(text: str) -> str:
    """Logical-order text with Arabic letters replaced by their contextual presentation forms."""
    letters, ligatures = _tables()
    forms = arabic_forms(text)
    n = len(forms)
    out: List[str] = []
    i = 0
    while i < n:
        ch, form = forms[i]
        if not form:
            out.append(ch)
            i += 1
            continue
        if ch == "ل":                                            # lam followed (marks aside) by an alef: one ligature
            j = i + 1
            marks = []
            while j < n and _is_mark(forms[j][0]):
                marks.append(forms[j][0])
                j += 1
            if j < n and (ch, forms[j][0]) in ligatures:
                lig = ligatures[(ch, forms[j][0])]
                joined = form in (FINAL, MEDIAL)
                out.append(lig[FINAL] if joined and FINAL in lig else lig[ISOLATED])
                out.extend(marks)
                i = j + 1
                continue
        out.append(letters[ch].get(form, letters[ch].get(ISOLATED, ch)))
        i += 1
    return "".join(out)


def _direction(ch: str) -> str:
    b = unicodedata.bidirectional(ch)
    if b in ("R", "AL"):
        return "R"
    if b == "L":
        return "L"
    if b in ("EN", "AN"):
        return "N"                                                     # numbers: left to right, inside either kind of run
    return ""                                                          # neutral or weak


def base_direction(text: str) -> str:
    for ch in text:
        d = _direction(ch)
        if d in ("L", "R"):
            return d
    return "L"


def visual_indices(text: str, base: str = "") -> List[Tuple[int, bool]]:
    """Drawing order of one line: (index into ``text``, whether that character is drawn mirrored), left to right."""
    base = base or base_direction(text)
    n = len(text)
    kinds = [_direction(c) for c in text]
    # numbers take the direction of the run they stand in (the last strong character before them, else the base)
    level = [""] * n
    last = base
    for i, k in enumerate(kinds):
        if k in ("L", "R"):
            last = k
            level[i] = k
        elif k == "N":
            level[i] = "RN" if last == "R" else "L"
    # neutrals: between two characters of one direction they join it, otherwise they take the base direction
    i = 0
    while i < n:
        if level[i]:
            i += 1
            continue
        j = i
        while j < n and not level[j]:
            j += 1
        left = level[i - 1][0] if i > 0 else base
        right = level[j][0] if j < n else base
        fill = left if left == right else base
        for k in range(i, j):
            level[k] = fill
        i = j
    # runs of one direction ("RN" = digits inside a right-to-left run: part of that run, kept in reading order)
    runs: List[List[Tuple[int, bool]]] = []
    i = 0
    while i < n:
        d = level[i][0]
        j = i
        while j < n and level[j][0] == d:
            j += 1
        seg = [(k, False) for k in range(i, j)]
        if d == "R":
            pieces, k = [], i
            while k < j:                                               # reverse, but keep each number as written
                if level[k] == "RN":
                    m = k
                    while m < j and level[m] == "RN":
                        m += 1
                    pieces.append([(q, False) for q in range(k, m)])
                    k = m
                else:
                    pieces.append([(k, text[k] in _MIRROR)])
                    k += 1
            seg = [item for piece in reversed(pieces) for item in piece]
        runs.append(seg)
        i = j
    if base == "R":
        runs.reverse()
    return [item for seg in runs for item in seg]


def visual_order(text: str, base: str = "") -> str:
    """The characters of one line in left-to-right drawing order."""
    return "".join(_MIRROR[text[i]] if mirrored else text[i] for i, mirrored in visual_indices(text, base))


def layout_line(text: str, base: str = "") -> str:
    """Shape, then reorder: what to hand to the rasteriser glyph by glyph, left to right."""
    return visual_order(shape_arabic(text), base or base_direction(text))
