"""Reading text lines with a convolutional-recurrent network and the CTC loss: lines of 3 to 7 characters drawn in a
seven-segment face (digits and the letters that face can show) with jitter and noise; a small CNN turns the image into
a sequence of column features, a bidirectional GRU reads it, and connectionist temporal classification aligns the
output with the text, so no character positions are ever labelled. On a GPU the convolutions, the recurrent cells and
the CTC loss all run on the package's kernels.

    python samples/ocr.py [--device cuda]

Reference: samples/Idrak.Samples.Ocr/Program.cs (a per-character CNN plus a segmenter there; the same task, lines in and
text out, is solved here without the segmenter).
"""
import argparse
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.nn import layers as L  # noqa: E402
from idrak_b200.nn.losses import ctc  # noqa: E402

SEGMENTS = {"0": "abcdef", "1": "bc", "2": "abdeg", "3": "abcdg", "4": "bcfg", "5": "acdfg", "6": "acdefg", "7": "abc",
            "8": "abcdefg", "9": "abcdfg", "A": "abcefg", "C": "adef", "E": "adefg", "F": "aefg", "H": "bcefg",
            "L": "def", "P": "abefg", "U": "bcdef"}
ALPHABET = "".join(SEGMENTS)                 # class k + 1 is ALPHABET[k]; class 0 is the CTC blank
HEIGHT, CELL = 14, 9


def glyph(ch: str) -> torch.Tensor:
    """A HEIGHT x CELL drawing of one character."""
    img = torch.zeros(HEIGHT, CELL)
    on = SEGMENTS[ch]
    top, mid, bot, left, right = 1, HEIGHT // 2, HEIGHT - 2, 1, CELL - 3
    if "a" in on:
        img[top, left:right + 1] = 1
    if "g" in on:
        img[mid, left:right + 1] = 1
    if "d" in on:
        img[bot, left:right + 1] = 1
    if "f" in on:
        img[top:mid + 1, left] = 1
    if "b" in on:
        img[top:mid + 1, right] = 1
    if "e" in on:
        img[mid:bot + 1, left] = 1
    if "c" in on:
        img[mid:bot + 1, right] = 1
    return img


GLYPHS = {ch: glyph(ch) for ch in ALPHABET}


def render(text: str, width: int, g: torch.Generator) -> torch.Tensor:
    """The line as a HEIGHT x width image: glyphs side by side with a random gap, shifted, blurred a little, noisy."""
    img = torch.zeros(HEIGHT, width)
    x = int(torch.randint(0, 4, (), generator=g))
    for ch in text:
        if x + CELL > width:
            break
        img[:, x:x + CELL] = torch.maximum(img[:, x:x + CELL], GLYPHS[ch])
        x += CELL - 1 + int(torch.randint(0, 3, (), generator=g))
    img = torch.roll(img, int(torch.randint(-1, 2, (), generator=g)), 0)
    img = 0.7 * img + 0.15 * (torch.roll(img, 1, 1) + torch.roll(img, -1, 1))
    return (img + 0.1 * torch.randn(HEIGHT, width, generator=g)).clamp(0, 1)


def dataset(count: int, seed: int, max_chars: int = 7):
    g = torch.Generator().manual_seed(seed)
    width = 4 + max_chars * (CELL + 2)
    texts, images = [], []
    for _ in range(count):
        n = int(torch.randint(3, max_chars + 1, (), generator=g))
        text = "".join(ALPHABET[int(k)] for k in torch.randint(0, len(ALPHABET), (n,), generator=g))
        texts.append(text)
        images.append(render(text, width, g))
    targets = torch.zeros(count, max_chars, dtype=torch.long)
    for i, t in enumerate(texts):
        targets[i, :len(t)] = torch.tensor([ALPHABET.index(c) + 1 for c in t])
    return torch.stack(images)[:, None], targets, torch.tensor([len(t) for t in texts]), texts


class LineReader(nn.Module):
    """CNN over the image (height pooled away, width halved), bidirectional GRU over the columns, one score row per
    column and class."""

    def __init__(self, classes: int, hidden: int = 48):
        super().__init__()
        self.features = nn.Sequential(L.Conv2d(1, 16, 3, padding=1), nn.ReLU(), L.MaxPool2d((2, 2)),
                                      L.Conv2d(16, 32, 3, padding=1), nn.ReLU(), L.MaxPool2d((HEIGHT // 2, 1)))
        self.rnn = L.Recurrent("gru", 32, hidden, sequences=True, bidirectional=True)
        self.head = L.Linear(2 * hidden, classes)

    def forward(self, images):
        f = self.features(images)                          # [N, 32, 1, W / 2]
        seq = f.squeeze(2).transpose(1, 2)                 # [N, T, 32]
        return self.head(self.rnn(seq))                    # [N, T, classes]


def greedy_text(scores: torch.Tensor):
    """Collapse repeats, drop blanks."""
    out = []
    for row in scores.argmax(-1).tolist():
        chars, last = [], 0
        for k in row:
            if k != last and k != 0:
                chars.append(ALPHABET[k - 1])
            last = k
        out.append("".join(chars))
    return out


def main(steps: int = 600, device: str = "cpu", quiet: bool = False, train_lines: int = 1500) -> dict:
    torch.manual_seed(0)
    x, targets, lengths, _ = dataset(train_lines, 1)
    xt, _, _, texts = dataset(200, 2)
    model = LineReader(len(ALPHABET) + 1).to(device)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    g = torch.Generator().manual_seed(7)
    for step in range(steps):
        idx = torch.randint(0, len(x), (64,), generator=g)
        scores = model(x[idx].to(device))                                   # [N, T, C]
        log_probs = torch.log_softmax(scores.float(), -1).transpose(0, 1)   # [T, N, C]
        frames = torch.full((len(idx),), log_probs.shape[0], dtype=torch.long)
        loss = ctc(log_probs, targets[idx].to(device), frames.to(device), lengths[idx].to(device))
        opt.zero_grad()
        loss.backward()
        nn.utils.clip_grad_norm_(model.parameters(), 5.0)
        opt.step()
        if not quiet and (step + 1) % 50 == 0:
            print(f"step {step + 1:4d}  ctc loss per character {float(loss.detach()):.4f}")
    model.eval()
    with torch.no_grad():
        read = greedy_text(model(xt.to(device)).float().cpu())
    exact = sum(a == b for a, b in zip(read, texts)) / len(texts)
    chars = sum(sum(p == q for p, q in zip(a, b)) for a, b in zip(read, texts)) / sum(len(t) for t in texts)
    if not quiet:
        for a, b in list(zip(texts, read))[:8]:
            print(f"  {a:8s} read as {b}")
        print(f"lines read exactly {exact:.3f}, characters in place {chars:.3f}")
    return {"exact": exact, "characters": chars, "final_loss": float(loss.detach())}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=600)
    a = ap.parse_args()
    main(a.steps, a.device)
