"""Retrieval: cut documents into overlapping chunks, index them by BM25 and by vectors, fuse the two rankings, and
build the augmented chat messages a generator would answer from.

    python samples/rag.py "Which kernel sums gradients?"

The sample embeds with hashed character trigrams so that it runs without a model; pass any `embed(texts) -> vectors`
(an `EmbedModel` of the inference engine, for one) to `VectorIndex.build` in real use.

Reference: samples/Idrak.Samples.Rag/Program.cs.
"""
import os
import sys
import zlib

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.rag import VectorIndex, augment, chunks_of  # noqa: E402
from idrak_b200.rag.bm25 import Bm25Index, reciprocal_rank_fusion  # noqa: E402

DOCUMENTS = [
    ("gemm.txt", "The matrix product kernel stages operand tiles in shared memory with bulk tensor copies and accumulates "
                 "in tensor memory. The epilogue adds the bias and applies the activation before the store."),
    ("dp.txt", "The data-parallel step sums gradients with a reduce-scatter kernel that loads the peers' buckets over "
               "NVLink in a fixed rank order, so every rank sees the same bits. AdamW then updates the owned shard."),
    ("serve.txt", "The serving engine admits requests under a prefill token budget, keeps key and value blocks in a paged "
                  "pool, and preempts the youngest sequence when blocks run out."),
]


def embed(texts, dim: int = 256):
    rows = torch.zeros(len(texts), dim)
    for r, t in enumerate(texts):
        t = t.lower()
        for i in range(len(t) - 2):
            rows[r, zlib.crc32(t[i: i + 3].encode()) % dim] += 1.0
    return rows


def main(question: str = "Which kernel sums gradients?", quiet: bool = False) -> dict:
    chunks = chunks_of(DOCUMENTS, size=160, overlap=30)
    lexical, vectors = Bm25Index(chunks), VectorIndex.build(chunks, embed)
    a, b = lexical.search(question, k=4), vectors.search(embed([question])[0], k=4)
    fused = reciprocal_rank_fusion([a, b], k=2)
    messages = augment(question, fused)
    if not quiet:
        for h in fused:
            print(f"{h.score:.4f}  {h.chunk.source}: {h.chunk.text[:70]}...")
        print(messages[-1]["content"][:300])
    return {"sources": [h.chunk.source for h in fused], "messages": messages}


if __name__ == "__main__":
    main(*sys.argv[1:2])
