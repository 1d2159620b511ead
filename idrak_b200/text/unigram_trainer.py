"""Unigram language-model tokenizer training (the SentencePiece algorithm) in plain Python.

1. words = text split on whitespace, each prefixed with the meta space; counted.
2. seed pieces = every substring (up to ``max_piece_length`` characters) seen at least twice, ranked by
   frequency x length, cut to ``seed_factor`` x the target size, plus every single character.
3. EM: the E step runs forward-backward over each word's lattice of pieces and collects expected piece counts; the
   M step sets score = digamma(count) - digamma(total) (the Bayesian variant, which starves rare pieces).
4. pruning: a piece's loss is what the corpus likelihood drops by when it is removed and its occurrences fall back to
   its best alternative segmentation; the ``shrink`` fraction with the highest loss survives (single characters
   always do), until the target size is reached.

Returns (piece, score) pairs, best first after the required characters; ``train_unigram`` wraps them into a tokenizer.

Reference: UnigramTrainer.cs (src/Idrak/Models/Tokenizers).
"""
from __future__ import annotations

import math
from collections import Counter
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

META = "▁"


def _digamma(x: float) -> float:
    r = 0.0
    while x < 7:
        r -= 1.0 / x
        x += 1
    x -= 0.5
    xx = 1.0 / x
    xx2 = xx * xx
    xx4 = xx2 * xx2
    return r + math.log(x) + (1.0 / 24.0) * xx2 - (7.0 / 960.0) * xx4 + (31.0 / 8064.0) * xx4 * xx2 - (127.0 / 30720.0) * xx4 * xx4


def _logaddexp(a: float, b: float) -> float:
    if a == -math.inf:
        return b
    if b == -math.inf:
        return a
    m = a if a > b else b
    return m + math.log(math.exp(a - m) + math.exp(b - m))


class _Lattice:
    """All pieces of the vocabulary that occur in one word: edges (start, end, piece)."""

    def __init__(self, word: str, scores: Dict[str, float], max_len: int):
        self.n = len(word)
        self.begin: List[List[Tuple[int, str, float]]] = [[] for _ in range(self.n + 1)]
        for i in range(self.n):
            for j in range(i + 1, min(self.n, i + max_len) + 1):
                p = word[i:j]
                s = scores.get(p)
                if s is not None:
                    self.begin[i].append((j, p, s))

    def viterbi(self, skip: Optional[str] = None) -> Tuple[float, List[str]]:
        best = [-math.inf] * (self.n + 1)
        back: List[Optional[Tuple[int, str]]] = [None] * (self.n + 1)
        best[0] = 0.0
        for i in range(self.n):
            if best[i] == -math.inf:
                continue
            for j, p, s in self.begin[i]:
                if p == skip:
                    continue
                if best[i] + s > best[j]:
                    best[j], back[j] = best[i] + s, (i, p)
        if best[self.n] == -math.inf:
            return -math.inf, []
        out, j = [], self.n
        while j > 0:
            i, p = back[j]
            out.append(p)
            j = i
        return best[self.n], out[::-1]

    def expected(self, weight: float, into: Dict[str, float]) -> float:
        """Adds weight x P(piece used) for every edge; returns weight x log Z."""
        alpha = [-math.inf] * (self.n + 1)
        beta = [-math.inf] * (self.n + 1)
        alpha[0] = 0.0
        for i in range(self.n):
            if alpha[i] == -math.inf:
                continue
            for j, _, s in self.begin[i]:
                alpha[j] = _logaddexp(alpha[j], alpha[i] + s)
        beta[self.n] = 0.0
        for i in range(self.n - 1, -1, -1):
            for j, _, s in self.begin[i]:
                if beta[j] != -math.inf:
                    beta[i] = _logaddexp(beta[i], s + beta[j])
        z = alpha[self.n]
        if z == -math.inf:
            return 0.0
        for i in range(self.n):
            if alpha[i] == -math.inf:
                continue
            for j, p, s in self.begin[i]:
                if beta[j] != -math.inf:
                    into[p] = into.get(p, 0.0) + weight * math.exp(alpha[i] + s + beta[j] - z)
        return weight * z


def count_words(texts: Iterable[str]) -> Counter:
    words: Counter = Counter()
    for t in texts:
        for w in t.split():
            words[META + w] += 1
    return words


def train_unigram_pieces(texts: Iterable[str], vocab_size: int, max_piece_length: int = 16, seed_factor: int = 8,
                         shrink: float = 0.75, em_rounds: int = 2, required: Sequence[str] = ()) -> List[Tuple[str, float]]:
    words = count_words(texts)
    if not words:
        raise ValueError("unigram training needs some text")
    chars: Counter = Counter()
    subs: Counter = Counter()
    for w, c in words.items():
        for i in range(len(w)):
            chars[w[i]] += c
            for j in range(i + 2, min(len(w), i + max_piece_length) + 1):
                subs[w[i:j]] += c
    for r in required:
        chars.setdefault(r, 1)
    if vocab_size < len(chars):
        raise ValueError(f"vocabulary of {vocab_size} cannot hold the {len(chars)} distinct characters")
    seeds = sorted(((p, c) for p, c in subs.items() if c >= 2), key=lambda pc: (-pc[1] * len(pc[0]), pc[0]))
    seeds = seeds[: max(vocab_size * seed_factor, vocab_size + 16)]
    counts: Dict[str, float] = {p: float(c) for p, c in seeds}
    counts.update({ch: float(c) for ch, c in chars.items()})
    total = sum(counts.values())
    scores = {p: math.log(c / total) for p, c in counts.items()}
    word_list = sorted(words.items())

    def em(scores: Dict[str, float]) -> Dict[str, float]:
        max_len = max(len(p) for p in scores)
        exp: Dict[str, float] = {}
        for w, c in word_list:
            _Lattice(w, scores, max_len).expected(float(c), exp)
        # pieces with vanishing expected counts leave (characters stay whatever their count)
        kept = {p: v for p, v in exp.items() if v >= 0.5 or len(p) == 1}
        for ch in chars:
            kept.setdefault(ch, 1e-3)
        tot = sum(kept.values())
        dg = _digamma(tot)
        return {p: _digamma(max(v, 1e-3)) - dg for p, v in kept.items()}

    while True:
        for _ in range(em_rounds):
            scores = em(scores)
        if len(scores) <= vocab_size:
            break
        # loss of removing each multi-character piece
        max_len = max(len(p) for p in scores)
        usage: Dict[str, float] = {}
        for w, c in word_list:
            _, seg = _Lattice(w, scores, max_len).viterbi()
            for p in seg:
                usage[p] = usage.get(p, 0.0) + c
        tot_usage = sum(usage.values()) or 1.0
        losses: List[Tuple[float, str]] = []
        for p, s in scores.items():
            if len(p) == 1:
                continue
            f = usage.get(p, 0.0)
            if f == 0:
                losses.append((0.0, p))
                continue
            alt, seg = _Lattice(p, scores, max_len).viterbi(skip=p)
            if not seg:
                losses.append((math.inf, p))          # nothing else spells it: keep
                continue
            losses.append((f / tot_usage * (s - alt), p))
        losses.sort(key=lambda lp: (-lp[0], lp[1]))
        singles = [p for p in scores if len(p) == 1]
        room = max(vocab_size - len(singles), 0)
        keep_n = max(room, int(len(losses) * shrink)) if len(losses) * shrink > room else room
        kept = set(singles) | {p for _, p in losses[:keep_n]}
        scores = {p: s for p, s in scores.items() if p in kept}
    norm = math.log(sum(math.exp(s) for s in scores.values()))
    out = sorted(((p, s - norm) for p, s in scores.items()), key=lambda ps: (-ps[1], ps[0]))
    return out


def train_unigram(texts: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = ("<unk>", "<s>", "</s>"),
                  byte_fallback: bool = False, **options):
    """Trains and returns a ready tokenizer (Metaspace pre-tokenizer, Unigram model). ``vocab_size`` counts the special
    tokens (and the 256 byte pieces with ``byte_fallback``). ``tokenizer.model`` holds the SentencePiece form."""
    from .sentencepiece_model import from_unigram, to_tokenizer
    reserved = len(special_tokens) + (256 if byte_fallback else 0)
    pieces = train_unigram_pieces(list(texts), vocab_size - reserved, **options)
    model = from_unigram(pieces, special_tokens, byte_fallback)
    tok = to_tokenizer(model)
    tok.model = model
    return tok
