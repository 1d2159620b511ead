"""Synthetic page layout: wrap text into lines inside margins, place the glyph outlines, rasterise the whole page in
one pass and return the page image together with the word boxes (the labels an OCR / layout model trains on).

    page = compose_page(font, text, width=1240, height=1754, font_size=28, device="cuda")
    page.image      # uint8 [H, W, 1], dark ink on a light page
    page.words      # [WordBox(text, x0, y0, x1, y1, line), ...]

Reference: the reference's page synthesiser (src/Idrak.Imaging/ShapesLayout.cs and the text layouts its OCR samples
use: wrapped paragraphs, alignment, per-word boxes as ground truth).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .font import TrueTypeFont
from .raster import Path, rasterize, rect


@dataclass
class WordBox:
    text: str
    x0: float
    y0: float
    x1: float
    y1: float
    line: int


@dataclass
class Page:
    image: torch.Tensor                 # uint8 [H, W, 1]
    words: List[WordBox] = field(default_factory=list)
    lines: List[str] = field(default_factory=list)


def wrap(font: TrueTypeFont, text: str, size: float, max_width: float) -> List[List[str]]:
    """Greedy word wrap; blank lines in the text start new paragraphs. A word wider than the line stands alone."""
    space = font.measure(" ", size)[0]
    out: List[List[str]] = []
    for paragraph in text.split("\n"):
        words = paragraph.split()
        if not words:
            out.append([])
            continue
        cur: List[str] = []
        cur_w = 0.0
        for w in words:
            ww = font.measure(w, size)[0]
            if cur and cur_w + space + ww > max_width:
                out.append(cur)
                cur, cur_w = [w], ww
            else:
                cur_w = ww if not cur else cur_w + space + ww
                cur.append(w)
        out.append(cur)
    return out


def compose_page(font: TrueTypeFont, text: str, width: int, height: int, font_size: float = 24.0,
                 margins: Tuple[float, float, float, float] = (60, 60, 60, 60), line_spacing: float = 1.25,
                 align: str = "left", ink: int = 20, paper: int = 245, device: Optional[str] = None,
                 rules: Sequence[Tuple[float, float, float, float]] = ()) -> Page:
    """Lay ``text`` out on a ``width`` x ``height`` page. ``margins`` = (left, top, right, bottom); ``align`` one of
    left / right / center / justify; ``rules`` are filled rectangles (x0, y0, x1, y1) such as table lines. Text that
    does not fit below the bottom margin is dropped."""
    if align not in ("left", "right", "center", "justify"):
        raise ValueError("align must be left, right, center or justify")
    left, top, right, bottom = margins
    usable = width - left - right
    scale = font_size / font.units_per_em
    ascent, descent = font.ascender * scale, -font.descender * scale
    step = (ascent + descent) * line_spacing
    space = font.measure(" ", font_size)[0]
    outline = Path()
    words: List[WordBox] = []
    lines_out: List[str] = []
    baseline = top + ascent
    wrapped = wrap(font, text, font_size, usable)
    for li, line in enumerate(wrapped):
        if baseline + descent > height - bottom:
            break
        if line:
            widths = [font.measure(w, font_size)[0] for w in line]
            natural = sum(widths) + space * (len(line) - 1)
            gap = space
            x = left
            last_of_paragraph = li + 1 >= len(wrapped) or not wrapped[li + 1]
            if align == "right":
                x = left + usable - natural
            elif align == "center":
                x = left + (usable - natural) / 2
            elif align == "justify" and len(line) > 1 and not last_of_paragraph:
                gap = (usable - sum(widths)) / (len(line) - 1)
            for w, ww in zip(line, widths):
                outline.contours += font.text_path(w, font_size, x=x, baseline=baseline).contours
                words.append(WordBox(w, x, baseline - ascent, x + ww, baseline + descent, len(lines_out)))
                x += ww + gap
        lines_out.append(" ".join(line))
        baseline += step
    for r in rules:
        outline.contours += rect(*r).contours
    cov = rasterize([outline], width, height, device=device, dtype=torch.float32)[0]
    image = (paper - cov * float(paper - ink)).round_().clamp_(0, 255).to(torch.uint8)[..., None]
    return Page(image, words, lines_out)
