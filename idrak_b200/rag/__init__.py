"""Retrieval-augmented generation: split documents into chunks, embed them, search by cosine similarity, build the
prompt that carries the retrieved passages.

    index = VectorIndex.build(chunks_of(texts, size=400, overlap=50), embed=lambda batch: engine.embed("m", batch))
    hits = index.search(embed([question])[0], k=4)
    messages = augment(question, hits)

The index is a dense matrix on the embedding tensor's device; a search is one GEMV / GEMM and a top-k.
Save / load keeps vectors as safetensors and the texts beside them as JSON lines.

Reference: the retrieval commands and store of the reference (src/Idrak.Text/Retrieval/*: chunking, embedding
store, cosine search, prompt assembly).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Sequence

import torch


@dataclass
class Chunk:
    text: str
    source: str = ""
    start: int = 0


@dataclass
class Hit:
    chunk: Chunk
    score: float
    index: int


def chunks_of(texts: Iterable, size: int = 400, overlap: int = 50) -> List[Chunk]:
    """Cut texts into chunks of about ``size`` characters on sentence / paragraph boundaries, each overlapping the
    previous by about ``overlap`` characters. ``texts``: strings or (source, text) pairs."""
    if overlap >= size:
        raise ValueError("overlap must be smaller than the chunk size")
    out: List[Chunk] = []
    for item in texts:
        source, text = item if isinstance(item, tuple) else ("", item)
        pieces = [p for p in re.split(r"(?<=[.!?])\s+|\n{2,}", text) if p.strip()]
        cur, cur_start, pos = "", 0, 0
        for piece in pieces:
            at = text.find(piece, pos)
            pos = at + len(piece) if at >= 0 else pos
            if cur and len(cur) + 1 + len(piece) > size:
                out.append(Chunk(cur, source, cur_start))
                tail = cur[-overlap:] if overlap else ""
                if " " in tail:
                    tail = tail[tail.find(" ") + 1:]       # start the overlap at a word
                cur, cur_start = (tail + " " + piece).strip(), max(at - len(tail), 0)
            else:
                if not cur:
                    cur_start = max(at, 0)
                cur = (cur + " " + piece).strip()
            while len(cur) > size * 2:                   # one giant sentence: cut it hard
                out.append(Chunk(cur[:size], source, cur_start))
                cur, cur_start = cur[size - overlap:], cur_start + size - overlap
        if cur:
            out.append(Chunk(cur, source, cur_start))
    return out


class VectorIndex:
    def __init__(self, vectors: torch.Tensor, chunks: Sequence[Chunk]):
        if vectors.shape[0] != len(chunks):
            raise ValueError("one vector per chunk")
        self.vectors = torch.nn.functional.normalize(vectors.float(), dim=-1)
        self.chunks = list(chunks)

    @classmethod
    def build(cls, chunks: Sequence[Chunk], embed: Callable[[List[str]], Sequence], batch: int = 32,
              device: Optional[str] = None) -> "VectorIndex":
        rows = []
        for i in range(0, len(chunks), batch):
            vecs = embed([c.text for c in chunks[i: i + batch]])
            rows.append(torch.as_tensor(vecs, dtype=torch.float32))
        v = torch.cat(rows) if rows else torch.zeros(0, 1)
        return cls(v.to(device) if device else v, chunks)

    def __len__(self) -> int:
        return len(self.chunks)

    def search(self, query: Sequence[float], k: int = 4, min_score: float = -1.0) -> List[Hit]:
        if len(self) == 0:
            return []
        q = torch.nn.functional.normalize(torch.as_tensor(query, dtype=torch.float32, device=self.vectors.device), dim=-1)
        scores = self.vectors @ q
        top = torch.topk(scores, min(k, len(self)))
        return [Hit(self.chunks[int(i)], float(s), int(i)) for s, i in zip(top.values, top.indices) if float(s) >= min_score]

    def add(self, chunks: Sequence[Chunk], vectors) -> None:
        v = torch.nn.functional.normalize(torch.as_tensor(vectors, dtype=torch.float32), dim=-1).to(self.vectors.device)
        self.vectors = torch.cat([self.vectors, v]) if len(self) else v
        self.chunks += list(chunks)

    def save(self, folder: str) -> None:
        from ..formats.safetensors import save_file
        os.makedirs(folder, exist_ok=True)
        save_file({"vectors": self.vectors.cpu()}, os.path.join(folder, "vectors.safetensors"),
                  metadata={"format": "idrak-index", "count": str(len(self))})
        with open(os.path.join(folder, "chunks.jsonl"), "w", encoding="utf-8") as f:
            for c in self.chunks:
                f.write(json.dumps({"text": c.text, "source": c.source, "start": c.start}, ensure_ascii=False) + "\n")

    @classmethod
    def load(cls, folder: str, device: Optional[str] = None) -> "VectorIndex":
        from ..formats.safetensors import load_file
        v = load_file(os.path.join(folder, "vectors.safetensors"))["vectors"]
        with open(os.path.join(folder, "chunks.jsonl"), "r", encoding="utf-8") as f:
            chunks = [Chunk(**json.loads(line)) for line in f if line.strip()]
        return cls(v.to(device) if device else v, chunks)


DEFAULT_INSTRUCTION = ("Answer the question using the passages below. If they do not contain the answer, say that you "
                       "do not know.")


def augment(question: str, hits: Sequence[Hit], instruction: str = DEFAULT_INSTRUCTION, max_chars: int = 6000) -> List[dict]:
    """Chat messages carrying the retrieved passages (numbered, with their sources) and the question."""
    parts, used = [], 0
    for n, h in enumerate(hits, 1):
        label = f"[{n}]" + (f" ({h.chunk.source})" if h.chunk.source else "")
        block = f"{label}\n{h.chunk.text}"
        if used + len(block) > max_chars and parts:
            break
        parts.append(block)
        used += len(block)
    context = "\n\n".join(parts) if parts else "(no passages found)"
    return [{"role": "system", "content": instruction},
            {"role": "user", "content": f"Passages:\n{context}\n\nQuestion: {question}"}]


from .bm25 import Bm25Index, reciprocal_rank_fusion, rerank  # noqa: E402
