"""Lexical retrieval and result fusion: a BM25 index over chunks, reciprocal-rank fusion of several rankings (lexical
+ vector), and reranking of a short list with a cross-encoder.

    lexical = Bm25Index(chunks)
    fused = reciprocal_rank_fusion([lexical.search(q, 20), vectors.search(embed(q), 20)], k=5)
    best = rerank(q, fused, score=lambda pairs: cross_encoder_scores(pairs))

Reference: the retrieval package of the reference (src/Idrak.Text/Retrieval: BM25, vector index, cross-encoder,
chunking, fusion).
"""
from __future__ import annotations

import math
import re
from collections import Counter
from typing import Callable, Dict, List, Sequence, Tuple

from . import Chunk, Hit

_WORD = re.compile(r"\w+", re.UNICODE)


def tokenize(text: str) -> List[str]:
    return _WORD.findall(text.lower())


class Bm25Index:
    """Okapi BM25 with the usual ``k1`` / ``b`` and the non-negative idf ``ln(1 + (N - n + 0.5) / (n + 0.5))``."""

    def __init__(self, chunks: Sequence[Chunk], k1: float = 1.5, b: float = 0.75):
        self.chunks, self.k1, self.b = list(chunks), k1, b
        self.postings: Dict[str, List[Tuple[int, int]]] = {}
        self.lengths: List[int] = []
        for i, c in enumerate(self.chunks):
            words = tokenize(c.text)
            self.lengths.append(len(words))
            for w, n in Counter(words).items():
                self.postings.setdefault(w, []).append((i, n))
        self.mean_length = sum(self.lengths) / max(len(self.lengths), 1)

    def __len__(self) -> int:
        return len(self.chunks)

    def search(self, query: str, k: int = 4) -> List[Hit]:
        scores: Dict[int, float] = {}
        N = len(self.chunks)
        for w in set(tokenize(query)):
            post = self.postings.get(w)
            if not post:
                continue
            idf = math.log(1.0 + (N - len(post) + 0.5) / (len(post) + 0.5))
            for i, tf in post:
                norm = tf + self.k1 * (1 - self.b + self.b * self.lengths[i] / max(self.mean_length, 1e-9))
                scores[i] = scores.get(i, 0.0) + idf * tf * (self.k1 + 1) / norm
        top = sorted(scores.items(), key=lambda kv: (-kv[1], kv[0]))[:k]
        return [Hit(self.chunks[i], s, i) for i, s in top]


def reciprocal_rank_fusion(rankings: Sequence[Sequence[Hit]], k: int = 4, constant: float = 60.0) -> List[Hit]:
    """Score of a chunk = sum over rankings of 1 / (constant + rank); chunks are matched by their index."""
    fused: Dict[int, float] = {}
    first: Dict[int, Hit] = {}
    for ranking in rankings:
        for rank, h in enumerate(ranking, 1):
            fused[h.index] = fused.get(h.index, 0.0) + 1.0 / (constant + rank)
            first.setdefault(h.index, h)
    top = sorted(fused.items(), key=lambda kv: (-kv[1], kv[0]))[:k]
    return [Hit(first[i].chunk, s, i) for i, s in top]


def rerank(query: str, hits: Sequence[Hit], score: Callable[[List[Tuple[str, str]]], Sequence[float]], k: int = 4) -> List[Hit]:
    """Order a short list by a pair scorer (a cross-encoder's relevance logit for (query, passage))."""
    if not hits:
        return []
    scores = list(score([(query, h.chunk.text) for h in hits]))
    order = sorted(range(len(hits)), key=lambda i: (-float(scores[i]), i))[:k]
    return [Hit(hits[i].chunk, float(scores[i]), hits[i].index) for i in order]
