"""Sequence classification where word order matters: the sentiment of short sentences in which "not" flips the next
word ("not good" is negative, "not bad" positive). A bag of words cannot tell them apart; an LSTM, a GRU and a small
Transformer can. Embedding, LSTM, GRU, PositionalEncoding and TransformerEncoderLayer through the network builder; on
a GPU the recurrent layers run the package's cell kernels.

    python samples/sentiment.py [--device cuda]

Reference: samples/Idrak.Samples.Sentiment/Program.cs.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn.builder import Network  # noqa: E402

GOOD = ["good", "great", "fine", "lovely", "fun"]
BAD = ["bad", "awful", "dull", "poor", "boring"]
FILLER = ["the", "movie", "was", "it", "is", "at", "all", "really", "plot", "acting", "<pad>", "not"]
WORDS = FILLER + GOOD + BAD
INDEX = {w: i for i, w in enumerate(WORDS)}
LENGTH = 8


def sentence(g: torch.Generator):
    """A sentence and its label (1 = positive): one opinion word, negated half of the time."""
    pick = lambda items: items[int(torch.randint(0, len(items), (), generator=g))]       # noqa: E731
    positive_word = bool(torch.rand((), generator=g) < 0.5)
    negated = bool(torch.rand((), generator=g) < 0.5)
    words = [pick(["the", "it"]), pick(["movie", "plot", "acting"]), pick(["was", "is"])]
    if bool(torch.rand((), generator=g) < 0.5):
        words.append("really")
    if negated:
        words.append("not")
    words.append(pick(GOOD if positive_word else BAD))
    if bool(torch.rand((), generator=g) < 0.3):
        words += ["at", "all"]
    return words, int(positive_word != negated)


def encode(words):
    ids = [INDEX[w] for w in words][:LENGTH]
    return ids + [INDEX["<pad>"]] * (LENGTH - len(ids))


def dataset(count: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    rows = [sentence(g) for _ in range(count)]
    return torch.tensor([encode(w) for w, _ in rows]), torch.tensor([label for _, label in rows])


def models():
    v = len(WORDS)
    return {
        "bag of words": lambda: _BagOfWords(v),
        "lstm": lambda: Network.tokens(LENGTH).embedding(v, 24).lstm(32).linear(2).build(),
        "gru": lambda: Network.tokens(LENGTH).embedding(v, 24).gru(32).linear(2).build(),
        "transformer": lambda: _Pooled(Network.tokens(LENGTH).embedding(v, 32).positional().transformer(4, 64).build(), 32),
    }


class _BagOfWords(torch.nn.Module):
    def __init__(self, v):
        super().__init__()
        self.table = torch.nn.Embedding(v, 2)

    def forward(self, ids):
        return self.table(ids).sum(1)


class _Pooled(torch.nn.Module):
    def __init__(self, body, dim):
        super().__init__()
        self.body, self.head = body, torch.nn.Linear(dim, 2)

    def forward(self, ids):
        return self.head(self.body(ids).mean(1))


def train(model, x, y, epochs, device):
    model.to(device)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(5)
    for _ in range(epochs):
        order = torch.randperm(len(x), generator=g)
        for i in range(0, len(x), 128):
            idx = order[i:i + 128]
            loss = torch.nn.functional.cross_entropy(model(x[idx].to(device)), y[idx].to(device))
            opt.zero_grad()
            loss.backward()
            opt.step()
    return model


def main(epochs: int = 12, device: str = "cpu", quiet: bool = False, only=None) -> dict:
    torch.manual_seed(0)
    x, y = dataset(2000, 1)
    xt, yt = dataset(500, 2)
    scores = {}
    for name, make in models().items():
        if only and name not in only:
            continue
        model = train(make(), x, y, epochs, device)
        model.eval()
        with torch.no_grad():
            scores[name] = float((model(xt.to(device)).argmax(-1).cpu() == yt).float().mean())
        if not quiet:
            print(f"{name:13s} held-out accuracy {scores[name]:.3f}")
    return scores


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--epochs", type=int, default=12)
    a = ap.parse_args()
    main(a.epochs, a.device)
