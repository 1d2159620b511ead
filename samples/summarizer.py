"""Text summarisation: short reports about matches (teams, place, day, goals) and one-sentence summaries. Two extractive
baselines pick a sentence from the report; the abstractive model, a small word-level decoder-only transformer, writes
the summary token by token. Training shows it "<report> <sum> <summary> <end>" with the loss masked on the report, so
it learns to write summaries, not reports - and the summary needs a comparison of the two scores that no single
sentence of the report contains.

    python samples/summarizer.py [--device cuda]

Reference: samples/Idrak.Samples.Summarizer/Program.cs.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402

TEAMS = ["lions", "owls", "bears", "hawks", "wolves", "foxes"]
PLACES = ["kelso", "perth", "oban", "ayr"]
DAYS = ["friday", "saturday", "sunday"]
IGNORE = -100


def report(g: torch.Generator):
    pick = lambda items: items[int(torch.randint(0, len(items), (), generator=g))]          # noqa: E731
    a = pick(TEAMS)
    b = pick([t for t in TEAMS if t != a])
    place, day = pick(PLACES), pick(DAYS)
    ga, gb = int(torch.randint(0, 6, (), generator=g)), int(torch.randint(0, 6, (), generator=g))
    sentences = [f"the {a} played the {b} in {place} on {day} .", f"the {b} scored {gb} goals .", f"the {a} scored {ga} goals ."]
    if ga == gb:
        summary = f"the {a} and the {b} drew {ga} {gb} in {place} ."
    else:
        w, l, gw, gl = (a, b, ga, gb) if ga > gb else (b, a, gb, ga)
        summary = f"the {w} beat the {l} {gw} {gl} in {place} ."
    return " ".join(sentences), summary


class Words:
    def __init__(self, texts):
        words = sorted({w for t in texts for w in t.split()})
        self.words = ["<pad>", "<sum>", "<end>"] + words
        self.index = {w: i for i, w in enumerate(self.words)}

    def encode(self, text):
        return [self.index[w] for w in text.split()]

    def decode(self, ids):
        return " ".join(self.words[i] for i in ids)


def overlap(a: str, b: str) -> float:
    """Unigram F1 between two sentences (a plain stand-in for ROUGE-1)."""
    x, y = a.split(), b.split()
    common = sum(min(x.count(w), y.count(w)) for w in set(x))
    if not common:
        return 0.0
    p, r = common / len(x), common / len(y)
    return 2 * p * r / (p + r)


def rows(pairs, vocab: Words, length: int):
    ids = torch.zeros(len(pairs), length, dtype=torch.long)
    targets = torch.full((len(pairs), length), IGNORE, dtype=torch.long)
    for i, (rep, summ) in enumerate(pairs):
        r, s = vocab.encode(rep), vocab.encode(summ)
        seq = r + [vocab.index["<sum>"]] + s + [vocab.index["<end>"]]
        ids[i, :len(seq)] = torch.tensor(seq)
        start = len(r)                                    # position of <sum>: it predicts the first summary word
        targets[i, start:len(seq) - 1] = torch.tensor(seq[start + 1:])
    return ids, targets


@torch.no_grad()
def write_summary(model, vocab: Words, rep: str, device, limit: int = 16) -> str:
    ids = vocab.encode(rep) + [vocab.index["<sum>"]]
    out = []
    for _ in range(limit):
        logits = model(torch.tensor([ids], device=device))[0, -1].float()
        nxt = int(logits.argmax())
        if nxt == vocab.index["<end>"]:
            break
        out.append(nxt)
        ids.append(nxt)
    return vocab.decode(out)


def main(steps: int = 300, device: str = "cpu", quiet: bool = False) -> dict:
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1)
    train = [report(g) for _ in range(3000)]
    held = [report(g) for _ in range(100)]
    vocab = Words([t for pair in train + held for t in pair])
    length = 48
    spec = DecoderSpec.llama(layers=2, dim=96, heads=4, kv_heads=4, ff_dim=256, vocab=len(vocab.words), max_positions=64)
    model = build_decoder(spec, seed=2).to(device)
    if device.startswith("cuda"):
        model = model.to(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.01)
    ids, targets = rows(train, vocab, length)
    loss = None
    for step in range(steps):
        idx = torch.randint(0, len(train), (64,), generator=g)
        loss = model.loss(ids[idx].to(device), targets[idx].to(device), ignore_index=IGNORE)
        opt.zero_grad()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        if not quiet and (step + 1) % 50 == 0:
            print(f"step {step + 1:4d}  loss on the summaries {float(loss.detach()):.4f}")
    model.eval()
    scores = {"first sentence": 0.0, "best sentence": 0.0, "model": 0.0}
    exact = 0
    for rep, summ in held:
        sentences = [s.strip() + " ." for s in rep.split(" .") if s.strip()]
        scores["first sentence"] += overlap(sentences[0], summ)
        scores["best sentence"] += max(overlap(s, summ) for s in sentences)       # an oracle over the report's sentences
        written = write_summary(model, vocab, rep, device)
        scores["model"] += overlap(written, summ)
        exact += written == summ
    scores = {k: v / len(held) for k, v in scores.items()}
    if not quiet:
        rep, summ = held[0]
        print("report :", rep)
        print("summary:", write_summary(model, vocab, rep, device), "| expected:", summ)
        for k, v in scores.items():
            print(f"{k:15s} word overlap {v:.3f}")
        print(f"summaries written exactly: {exact} of {len(held)}")
    return {"scores": scores, "exact": exact / len(held), "final_loss": float(loss.detach())}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=300)
    a = ap.parse_args()
    main(a.steps, a.device)
