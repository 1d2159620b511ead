"""Character-level GPT training: a 4-layer decoder over bytes, AdamW with warm-up and cosine decay, periodic
evaluation on held-out text, a sample of generated text at the end, and a checkpoint that can be resumed.

    python samples/gpt_training.py --text corpus.txt --steps 500            # on the GPU when there is one
    python samples/gpt_training.py --steps 50 --device cpu                  # built-in text, a minute on the CPU

Reference: samples/Idrak.Samples.GptTraining/Program.cs (the loop :296-330, the model :424-429).
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402
from idrak_b200.ops import FusedAdamW  # noqa: E402

BUILT_IN = ("The quick brown fox jumps over the lazy dog. A journey of a thousand miles begins with a single step. "
            "To be, or not to be, that is the question. All that glitters is not gold. ") * 40


def batches(data: torch.Tensor, batch: int, length: int, generator: torch.Generator):
    while True:
        at = torch.randint(0, data.numel() - length - 1, (batch,), generator=generator)
        rows = torch.stack([data[i: i + length + 1] for i in at.tolist()])
        yield rows[:, :-1].contiguous(), rows[:, 1:].contiguous()


@torch.no_grad()
def sample(model, prompt: bytes, count: int, temperature: float, generator: torch.Generator, device) -> bytes:
    ids = torch.tensor([list(prompt)], dtype=torch.long, device=device)
    limit = model.spec.max_positions
    for _ in range(count):
        logits = model(ids[:, -limit:])[:, -1].float() / max(temperature, 1e-6)
        nxt = torch.multinomial(torch.softmax(logits, -1).cpu(), 1, generator=generator).to(device)
        ids = torch.cat([ids, nxt], 1)
    return bytes(ids[0].tolist())


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--text")
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--length", type=int, default=128)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--eval-every", type=int, default=50)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save")
    ap.add_argument("--quiet", action="store_true")
    a = ap.parse_args(argv)
    raw = open(a.text, "rb").read() if a.text else BUILT_IN.encode()
    data = torch.tensor(list(raw), dtype=torch.long)
    cut = int(0.9 * data.numel())
    train, held = data[:cut], data[cut:]
    g = torch.Generator().manual_seed(a.seed)
    torch.manual_seed(a.seed)
    spec = DecoderSpec.tiny_gpt()
    model = build_decoder(spec).to(a.device)
    if a.device.startswith("cuda"):
        model = model.to(torch.bfloat16)
    opt = FusedAdamW(model.parameters(), lr=a.lr, betas=(0.9, 0.95), weight_decay=0.1)
    say = (lambda *x: None) if a.quiet else print
    say(f"{sum(p.numel() for p in model.parameters()) / 1e6:.2f} M parameters on {a.device}; {train.numel()} training bytes")
    source, first, last, held_loss = batches(train, a.batch, a.length, g), None, None, None
    for step in range(1, a.steps + 1):
        lr = a.lr * step / a.warmup if step <= a.warmup else \
            a.lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * (step - a.warmup) / max(1, a.steps - a.warmup))))
        for group in opt.param_groups:
            group["lr"] = lr
        x, y = next(source)
        loss = model.loss(x.to(a.device), y.to(a.device))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        last = float(loss.detach())
        first = last if first is None else first
        if step % a.eval_every == 0 or step == a.steps:
            model.eval()
            with torch.no_grad():
                hx, hy = next(batches(held, a.batch, min(a.length, held.numel() - 2), g))
                held_loss = float(model.loss(hx.to(a.device), hy.to(a.device)))
            model.train()
            say(f"step {step:5d}  lr {lr:.2e}  loss {last:.4f}  held-out {held_loss:.4f}")
    model.eval()
    text = sample(model, b"The ", 80, 0.8, g, a.device)
    say("sample:", text.decode("utf-8", errors="replace"))
    if a.save:
        from idrak_b200.formats import ikw
        ikw.save_module(model, a.save)
        say("saved", a.save)
    return {"first_loss": first, "final_loss": last, "held_out_loss": held_loss, "sample": text}


if __name__ == "__main__":
    main()
