"""Evaluation of language models: perplexity over a token stream (strided windows, each token scored once with as
much left context as the window allows), multiple-choice answer scoring by log-likelihood, and exact-match /
token-F1 for generated answers.

Reference: src/Idrak.Text/Evaluation.cs (perplexity with a stride, task accuracy), AnswerScorer.cs (summed or
length-normalised log-probability of each candidate continuation).
"""
from __future__ import annotations

import math
import re
from collections import Counter
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


@dataclass
class PerplexityResult:
    perplexity: float
    nll: float                     # mean negative log-likelihood per scored token, in nats
    tokens: int
    bits_per_token: float


@torch.no_grad()
def perplexity(model, tokens: Sequence[int], window: int = 1024, stride: Optional[int] = None, batch: int = 4,
               device: Optional[torch.device] = None) -> PerplexityResult:
    """Slide a ``window``-token context over ``tokens`` by ``stride`` (default: half a window); in every window only the
    tokens not scored by an earlier window count, so each token is predicted exactly once."""
    stride = stride or max(window // 2, 1)
    dev = device or next(model.parameters()).device
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    n = len(ids)
    if n < 2:
        raise ValueError("need at least two tokens")
    spans = []
    scored_to = 1                                         # token 0 has no context and is never scored
    begin = 0
    while scored_to < n:
        end = min(begin + window, n)
        spans.append((begin, end, scored_to))
        scored_to = end
        begin += stride
        if end == n:
            break
    total, count = 0.0, 0
    was = model.training
    model.eval()
    for i in range(0, len(spans), batch):
        group = spans[i: i + batch]
        width = max(e - b for b, e, _ in group)
        x = torch.zeros(len(group), width, dtype=torch.long)
        for r, (b, e, _) in enumerate(group):
            x[r, : e - b] = ids[b:e]
        logits = model(x.to(dev)).float()
        lp = F.log_softmax(logits[:, :-1, : ], -1)
        for r, (b, e, first) in enumerate(group):
            tgt = ids[b + 1: e].to(dev)
            row = lp[r, : e - b - 1].gather(-1, tgt[:, None])[:, 0]
            keep = row[first - b - 1:]
            total -= float(keep.sum())
            count += keep.numel()
    model.train(was)
    nll = total / max(count, 1)
    return PerplexityResult(math.exp(min(nll, 700.0)), nll, count, nll / math.log(2))


@torch.no_grad()
def score_continuations(model, prompt: Sequence[int], candidates: Sequence[Sequence[int]], normalise: bool = False,
                        device: Optional[torch.device] = None) -> List[float]:
    """Log-probability of each candidate continuation after the prompt (divided by its length with ``normalise``)."""
    dev = device or next(model.parameters()).device
    width = len(prompt) + max(len(c) for c in candidates)
    x = torch.zeros(len(candidates), width, dtype=torch.long)
    for r, c in enumerate(candidates):
        row = list(prompt) + list(c)
        x[r, : len(row)] = torch.tensor(row)
    lp = F.log_softmax(model(x.to(dev)).float(), -1)
    out = []
    for r, c in enumerate(candidates):
        pos = torch.arange(len(prompt) - 1, len(prompt) + len(c) - 1, device=dev)
        s = float(lp[r, pos, torch.tensor(list(c), device=dev)].sum())
        out.append(s / len(c) if normalise else s)
    return out


def multiple_choice_accuracy(model, items: Sequence[dict], normalise: bool = True) -> float:
    """``items``: dicts with ``prompt`` (token ids), ``choices`` (lists of token ids) and ``answer`` (index)."""
    right = 0
    for it in items:
        scores = score_continuations(model, it["prompt"], it["choices"], normalise)
        right += int(max(range(len(scores)), key=scores.__getitem__) == it["answer"])
    return right / max(len(items), 1)


def _normalise_answer(text: str) -> List[str]:
    text = re.sub(r"\b(a|an|the)\b", " ", text.lower())
    return re.sub(r"[^\w\s]", " ", text).split()


def exact_match(prediction: str, references: Sequence[str]) -> float:
    p = _normalise_answer(prediction)
    return float(any(p == _normalise_answer(r) for r in references))


def token_f1(prediction: str, references: Sequence[str]) -> float:
    p = _normalise_answer(prediction)
    best = 0.0
    for r in references:
        g = _normalise_answer(r)
        common = sum((Counter(p) & Counter(g)).values())
        if not p or not g:
            best = max(best, float(p == g))
        elif common:
            precision, recall = common / len(p), common / len(g)
            best = max(best, 2 * precision * recall / (precision + recall))
    return best
