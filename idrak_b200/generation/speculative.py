"""Speculative decoding: a small draft model proposes a few tokens, the target model checks them in one pass.

Greedy mode reproduces the target model's greedy output token for token: the target runs once over the last
accepted token plus the ``k`` proposals (a cached-prefix prefill that returns the logits of every position), the
longest prefix of proposals that equals the target's own arg-max is kept, and the target's next token comes for
free from the same pass. Sampled mode uses the accept / resample rule that leaves the target distribution unchanged
(accept proposal x with probability min(1, p(x) / q(x)), otherwise draw from the normalised positive part of p - q).
Rejected positions of either KV cache are simply overwritten by the next pass.

Reference: speculative decoding contract and TextGenerator.Speculative.cs (src/Idrak/Generation/TextGenerator.Speculative.cs).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..serve.runner import ModelRunner, PrefillItem


@dataclass
class SpeculativeResult:
    tokens: List[int] = field(default_factory=list)
    proposed: int = 0
    accepted: int = 0
    target_passes: int = 0

    @property
    def acceptance(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_pass(self) -> float:
        return len(self.tokens) / self.target_passes if self.target_passes else 0.0


class _Lane:
    """One model's cache for one sequence: blocks 0..n in order, and how many positions hold valid keys."""

    def __init__(self, model, max_tokens: int, block_size: int = 16):
        blocks = (max_tokens + block_size - 1) // block_size + 1
        self.runner = ModelRunner(model, blocks, block_size, max_batch=1)
        self.blocks = list(range(blocks))
        self.filled = 0
        self.vocab = model.spec.vocabulary

    def run(self, tokens: Sequence[int], start: int) -> torch.Tensor:
        """Compute ``tokens`` at positions start.. and return their logits ``[len(tokens), vocabulary]`` (fp32)."""
        logits = self.runner.prefill([PrefillItem(list(tokens), start, self.blocks)], all_logits=True)
        self.filled = start + len(tokens)
        return logits[:, : self.vocab].float()


class SpeculativeDecoder:
    def __init__(self, target, draft, max_tokens: int = 2048, lookahead: int = 4):
        if target.spec.vocabulary != draft.spec.vocabulary:
            raise ValueError("the draft model must share the target's vocabulary")
        self.target = _Lane(target.eval(), max_tokens)
        self.draft = _Lane(draft.eval(), max_tokens)
        self.lookahead = lookahead
        self.max_tokens = max_tokens

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos_token_ids: Sequence[int] = (),
                 temperature: float = 0.0, seed: int = 0) -> SpeculativeResult:
        res = SpeculativeResult()
        eos = set(int(t) for t in eos_token_ids)
        seq = [int(t) for t in prompt]
        if len(seq) + max_new_tokens + self.lookahead + 1 > self.max_tokens:
            raise ValueError("prompt + new tokens exceed the decoder's cache")
        gen = torch.Generator(device="cpu").manual_seed(seed)
        sample = temperature > 0.0

        def dist(logits):
            return torch.softmax(logits / max(temperature, 1e-6), -1)

        def pick(p):
            return int(torch.multinomial(p.cpu(), 1, generator=gen)) if sample else int(p.argmax())

        # both caches take the prompt except its last token, which opens the first verification pass
        if len(seq) > 1:
            self.target.run(seq[:-1], 0)
            self.draft.run(seq[:-1], 0)
        while len(res.tokens) < max_new_tokens:
            base = len(seq) - 1                          # position of the last accepted token
            k = min(self.lookahead, max_new_tokens - len(res.tokens) - 1)
            # ---- draft: k proposals, one token at a time
            proposals, q_rows = [], []
            feed = [seq[-1]]
            start = base
            for _ in range(max(k, 0)):
                lg = self.draft.run(feed, start)[-1]
                q = dist(lg) if sample else None
                t = pick(q) if sample else int(lg.argmax())
                proposals.append(t)
                q_rows.append(q)
                feed, start = [t], start + len(feed)
            # ---- target: one pass over the last accepted token and the proposals
            logits = self.target.run([seq[-1]] + proposals, base)
            res.target_passes += 1
            res.proposed += len(proposals)
            new: List[int] = []
            for i, t in enumerate(proposals):
                if sample:
                    p, q = dist(logits[i]), q_rows[i]
                    if float(torch.rand(1, generator=gen)) < min(1.0, float(p[t] / q[t].clamp_min(1e-30))):
                        new.append(t)
                        continue
                    rest = (p - q).clamp_min(0)
                    new.append(int(torch.multinomial((rest / rest.sum().clamp_min(1e-30)).cpu(), 1, generator=gen)))
                    break
                if int(logits[i].argmax()) == t:
                    new.append(t)
                    continue
                new.append(int(logits[i].argmax()))      # the target's own token replaces the first wrong proposal
                break
            else:
                new.append(pick(dist(logits[len(proposals)])) if sample else int(logits[len(proposals)].argmax()))
            res.accepted += len(new) - 1                 # the last new token is the target's own (correction or bonus)
            for t in new:
                seq.append(t)
                res.tokens.append(t)
                if t in eos or len(res.tokens) >= max_new_tokens:
                    return res
            # the draft's cache holds proposals up to base + k; what was rejected gets overwritten on the next pass,
            # but a fully accepted run needs the last proposal's keys, which the draft has not computed yet
            if len(new) == len(proposals) + 1 and proposals:
                self.draft.run([proposals[-1]], base + len(proposals))
        return res
