"""The small CPU configuration: a 4-layer GPT (d 128, 4 heads, MLP 512 GELU, LayerNorm, learned positions, byte
vocabulary, 128 positions), batch 8, token ids uniform in [0, 256) from a seed, AdamW lr 3e-4, 100 steps of
next-token cross-entropy in fp32 on the CPU. Prints tokens per second and the final loss as one JSON line.

    python -m idrak_b200.diag.tiny_gpt_cpu                 # this package's model and optimizer (CPU statements of the ops)
    python -m idrak_b200.diag.tiny_gpt_cpu --impl torch    # the same model written with library modules

Reference: the GptTraining sample (samples/Idrak.Samples.GptTraining/Program.cs:296-330, spec :424-429), which mirrors a
PyTorch script step for step.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["idrak_b200", "torch"], default="idrak_b200")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    g = torch.Generator().manual_seed(a.seed)
    data = torch.randint(0, 256, (a.steps, a.batch, 129), generator=g)
    if a.impl == "torch":
        import os
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        from baseline.torch_gpt2 import GPT2
        model = GPT2(4, 128, 4, 256, 128)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
        step_loss = lambda ids, tgt: model(ids, tgt)
    else:
        from ..models import DecoderSpec, build_decoder
        from ..ops import FusedAdamW
        model = build_decoder(DecoderSpec.tiny_gpt(), seed=a.seed)
        opt = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
        step_loss = lambda ids, tgt: model.loss(ids, tgt)
    losses = []
    t0 = time.perf_counter()
    for s in range(a.steps):
        b = data[s]
        loss = step_loss(b[:, :-1].contiguous(), b[:, 1:].contiguous())
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()))
    dt = time.perf_counter() - t0
    print(json.dumps({"metric": "train tokens/s (tiny GPT, CPU fp32)", "impl": a.impl, "value": round(a.steps * a.batch * 128 / dt, 1),
                      "unit": "tokens/s", "steps": a.steps, "first_loss": round(losses[0], 4), "final_loss": round(losses[-1], 4),
                      "seconds": round(dt, 2), "threads": torch.get_num_threads(),
                      "config": "4L d128 4 heads ff512 GELU, vocab 256, seq 128, batch 8, AdamW 3e-4"}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
