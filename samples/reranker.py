"""Two-stage retrieval: BM25 shortlists, a cross-encoder-style scorer reorders the shortlist. The scorer here counts
shared word stems weighted by rarity so the sample runs without a model; pass an engine's scoring model in real use.

    python samples/reranker.py "how are gradients summed across GPUs"

Reference: samples/Idrak.Samples.ReRanker/Program.cs.
"""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.rag import chunks_of  # noqa: E402
from idrak_b200.rag.bm25 import Bm25Index, rerank  # noqa: E402

DOCUMENTS = [
    ("optimizer.txt", "AdamW keeps two moments per weight. The sharded optimizer updates only the slice a GPU owns."),
    ("collective.txt", "Gradients are summed across GPUs by a reduce-scatter: every GPU adds its slice of all peers' buckets."),
    ("cache.txt", "The key value cache is paged; a block table maps a sequence's positions to blocks."),
    ("summing.txt", "Column sums of a matrix give the bias gradient; they are summed by a two-pass kernel."),
]


def stems(text: str):
    return [w.strip(".,;:?!").lower()[:5] for w in text.split() if len(w) > 2]


def make_scorer(corpus):
    seen = {}
    for _, text in corpus:
        for s in set(stems(text)):
            seen[s] = seen.get(s, 0) + 1

    def score(pairs):
        out = []
        for query, passage in pairs:
            q, p = set(stems(query)), stems(passage)
            out.append(sum(math.log(1 + len(corpus) / seen.get(s, 1)) for s in set(p) if s in q) / math.sqrt(len(p) + 1))
        return out
    return score


def main(question: str = "how are gradients summed across GPUs", quiet: bool = False) -> dict:
    chunks = chunks_of(DOCUMENTS, size=200, overlap=0)
    shortlist = Bm25Index(chunks).search(question, k=4)
    best = rerank(question, shortlist, make_scorer(DOCUMENTS), k=2)
    out = {"shortlist": [h.chunk.source for h in shortlist], "reranked": [h.chunk.source for h in best]}
    if not quiet:
        print(out)
    return out


if __name__ == "__main__":
    main(*sys.argv[1:2])
