"""Beam search over the paged KV cache.

Every live beam owns a block table; a step decodes all beams as one batch, expands each by its ``width`` best
tokens, keeps the ``width`` best continuations overall, and gives every survivor its parent's cache by copying
blocks (whole-block copies, all layers at once). Finished hypotheses (end-of-sequence) leave the batch and are
ranked by length-normalised log-probability; ``early_stopping`` ends the search once ``width`` hypotheses are
finished and no live beam can still beat the worst of them.

Reference: BeamSearch (src/Idrak/Generation/BeamSearch.cs): length penalty, early stopping, n-best output.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..serve.runner import ModelRunner, PrefillItem


@dataclass
class Hypothesis:
    tokens: List[int]
    logprob: float
    score: float
    finished: bool


class BeamSearch:
    def __init__(self, model, width: int = 4, max_tokens: int = 1024, length_penalty: float = 1.0,
                 early_stopping: bool = True, block_size: int = 16):
        self.width, self.length_penalty, self.early_stopping = width, length_penalty, early_stopping
        self.block_size = block_size
        self.blocks_per_beam = (max_tokens + block_size - 1) // block_size
        # two sets of beam slots: survivors are written into the other set so a parent can feed several children
        self.runner = ModelRunner(model.eval(), 2 * width * self.blocks_per_beam, block_size, max_batch=width)
        self.vocab = model.spec.vocabulary
        self.max_tokens = max_tokens

    def _slot_blocks(self, side: int, beam: int) -> List[int]:
        first = (side * self.width + beam) * self.blocks_per_beam
        return list(range(first, first + self.blocks_per_beam))

    def _copy_cache(self, src: List[int], dst: List[int], length: int) -> None:
        n = (length + self.block_size - 1) // self.block_size
        s = torch.tensor(src[:n], device=self.runner.device)
        d = torch.tensor(dst[:n], device=self.runner.device)
        for k, v in zip(self.runner.k_cache, self.runner.v_cache):
            k[d] = k[s]
            v[d] = v[s]

    def _score(self, logprob: float, length: int) -> float:
        return logprob / (max(length, 1) ** self.length_penalty)

    @torch.no_grad()
    def search(self, prompt: Sequence[int], max_new_tokens: int, eos_token_ids: Sequence[int] = (),
               n_best: int = 1) -> List[Hypothesis]:
        W, dev = self.width, self.runner.device
        eos = set(int(t) for t in eos_token_ids)
        prompt = [int(t) for t in prompt]
        if len(prompt) + max_new_tokens > self.max_tokens:
            raise ValueError("prompt + new tokens exceed the search's cache")
        side = 0
        logits = self.runner.prefill([PrefillItem(prompt, 0, self._slot_blocks(side, 0))])[0, : self.vocab].float()
        lp = torch.log_softmax(logits, -1)
        top = torch.topk(lp, min(W, self.vocab))
        beams = []                                   # (tokens generated, logprob, slot)
        for j in range(top.indices.numel()):
            if j > 0:
                self._copy_cache(self._slot_blocks(side, 0), self._slot_blocks(side, j), len(prompt))
            beams.append(([int(top.indices[j])], float(top.values[j]), j))
        finished: List[Hypothesis] = []
        for step in range(1, max_new_tokens + 1):
            live = []
            for toks, l, slot in beams:
                if toks[-1] in eos or step == max_new_tokens:
                    finished.append(Hypothesis(toks, l, self._score(l, len(toks)), toks[-1] in eos))
                else:
                    live.append((toks, l, slot))
            finished.sort(key=lambda h: -h.score)
            finished = finished[: max(W, n_best)]
            if not live:
                break
            if self.early_stopping and len(finished) >= W:
                # a beam's log-probability only falls; the most its score can gain is the longest length's divisor
                best_possible = max(l / (max_new_tokens ** self.length_penalty) if self.length_penalty > 0 else l
                                    for _, l, _ in live)
                if best_possible <= finished[W - 1].score:
                    break
            pos = len(prompt) + len(live[0][0]) - 1   # every live beam has the same length
            last = torch.tensor([t[-1] for t, _, _ in live], dtype=torch.int32, device=dev)
            positions = torch.full((len(live),), pos, dtype=torch.int32, device=dev)
            table = torch.tensor([self._slot_blocks(side, s) for _, _, s in live], dtype=torch.int32, device=dev)
            lg = self.runner.decode(last, positions, table, max_len_hint=pos + 1)[:, : self.vocab].float()
            lp = torch.log_softmax(lg, -1)
            cand = torch.tensor([l for _, l, _ in live], device=dev)[:, None] + lp
            flat = torch.topk(cand.reshape(-1), min(W, cand.numel()))
            new_beams = []
            for j in range(flat.indices.numel()):
                parent, tok = divmod(int(flat.indices[j]), self.vocab)
                toks, _, slot = live[parent]
                self._copy_cache(self._slot_blocks(side, slot), self._slot_blocks(1 - side, j), pos + 1)
                new_beams.append((toks + [tok], float(flat.values[j]), j))
            beams, side = new_beams, 1 - side
        else:
            for toks, l, _ in beams:
                finished.append(Hypothesis(toks, l, self._score(l, len(toks)), toks[-1] in eos))
        finished.sort(key=lambda h: -h.score)
        return finished[:n_best]
