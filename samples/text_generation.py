"""A small GPT that learns to continue text: a character-level, decoder-only transformer trained on sentences from a
small grammar (or your own text), saved, then used to generate one character at a time. ``--benchmark`` compares three
ways of generating the same text: recomputing the whole prefix for every character, the engine's paged key / value
cache (decode steps replayed as CUDA graphs on a GPU), and several continuations batched together.

    python samples/text_generation.py [--corpus book.txt] [--device cuda] [--benchmark]

Reference: samples/Idrak.Samples.TextGeneration/Program.cs.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402
from idrak_b200.serve.engine import GenerationOptions, LLMEngine  # noqa: E402

SUBJECTS = ["the old wizard", "a young knight", "the quiet baker", "my neighbour", "the grey cat"]
VERBS = ["found", "lost", "painted", "carried", "followed", "remembered"]
OBJECTS = ["a silver key", "the long road", "an empty house", "the last letter", "a broken clock"]
ENDINGS = ["in the morning", "before the rain", "without a word", "near the river", "after the feast"]


def grammar_text(sentences: int, seed: int) -> str:
    g = torch.Generator().manual_seed(seed)
    pick = lambda items: items[int(torch.randint(0, len(items), (), generator=g))]          # noqa: E731
    return " ".join(f"{pick(SUBJECTS)} {pick(VERBS)} {pick(OBJECTS)} {pick(ENDINGS)}." for _ in range(sentences))


def train(text: str, steps: int, device: str, quiet: bool):
    data = torch.tensor(list(text.encode()), dtype=torch.long)
    spec = DecoderSpec.gpt2(layers=3, dim=96, heads=4, vocab=256, max_positions=128)
    model = build_decoder(spec, seed=0).to(device)
    if device.startswith("cuda"):
        model = model.to(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.01)
    g = torch.Generator().manual_seed(1)
    loss = None
    for step in range(steps):
        starts = torch.randint(0, data.numel() - 97, (32,), generator=g)
        x = torch.stack([data[s:s + 96] for s in starts]).to(device)
        y = torch.stack([data[s + 1:s + 97] for s in starts]).to(device)
        loss = model.loss(x, y)
        opt.zero_grad()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        if not quiet and (step + 1) % 50 == 0:
            print(f"step {step + 1:4d}  loss {float(loss.detach()):.4f}")
    return model.eval(), float(loss.detach())


@torch.no_grad()
def generate_recompute(model, prompt: bytes, count: int, device) -> bytes:
    """The whole prefix through the model for every new character (greedy)."""
    ids = list(prompt)
    for _ in range(count):
        window = ids[-model.spec.max_positions:]
        ids.append(int(model(torch.tensor([window], device=device))[0, -1].float().argmax()))
    return bytes(ids[len(prompt):])


def generate_engine(engine: LLMEngine, prompts, count: int, temperature: float, top_k: int, seed: int):
    opts = [GenerationOptions(temperature=temperature, top_k=top_k, top_p=1.0, repeat_penalty=1.0, max_tokens=count,
                              seed=seed + i) for i in range(len(prompts))]
    return [bytes(r.output) for r in engine.generate([list(p) for p in prompts], opts)]


def main(steps: int = 250, device: str = "cpu", corpus=None, prompt: str = "the old wizard", length: int = 80,
         temperature: float = 0.7, top_k: int = 0, samples: int = 1, benchmark: bool = False, quiet: bool = False,
         save=None) -> dict:
    text = open(corpus).read() if corpus else grammar_text(1500, 0)
    model, loss = train(text, steps, device, quiet)
    if save:
        from idrak_b200.formats import ikw
        ikw.save_module(model, save)
    engine = LLMEngine(model, num_blocks=256, block_size=16, max_batch=max(samples, 8))
    length = min(length, model.spec.max_positions - len(prompt) - 1)
    outs = generate_engine(engine, [prompt.encode()] * samples, length, temperature, top_k, seed=3)
    result = {"final_loss": loss, "continuations": [o.decode("utf-8", errors="replace") for o in outs]}
    if not quiet:
        for o in result["continuations"]:
            print(f"{prompt}|{o}")
    if benchmark:
        greedy = dict(temperature=0.0, top_k=0)
        t0 = time.perf_counter()
        a = generate_recompute(model, prompt.encode(), length, device)
        t1 = time.perf_counter()
        b = generate_engine(engine, [prompt.encode()], length, seed=0, **greedy)[0]
        t2 = time.perf_counter()
        many = generate_engine(engine, [prompt.encode()] * 8, length, seed=0, **greedy)
        t3 = time.perf_counter()
        result["benchmark"] = {"recompute_chars_per_s": length / (t1 - t0), "cache_chars_per_s": length / (t2 - t1),
                               "batched_chars_per_s": 8 * length / (t3 - t2), "same_text": a == b and all(m == b for m in many)}
        if not quiet:
            for k, v in result["benchmark"].items():
                print(f"{k:24s} {v if isinstance(v, bool) else round(v, 1)}")
    return result


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--corpus")
    ap.add_argument("--steps", type=int, default=250)
    ap.add_argument("--input", default="the old wizard")
    ap.add_argument("--length", type=int, default=80)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--samples", type=int, default=1)
    ap.add_argument("--benchmark", action="store_true")
    ap.add_argument("--save")
    a = ap.parse_args()
    main(a.steps, a.device, a.corpus, a.input, a.length, a.temperature, a.top_k, a.samples, a.benchmark, save=a.save)
