"""Serving throughput of the continuous-batching engine on one GPU with random weights of a given architecture.

    python -m idrak_b200.diag.serve_bench --layers 32 --dim 4096 --heads 32 --kv-heads 8 --ff 14336 \
        --vocab 128256 --requests 256 --prompt 512 --gen 128 --max-batch 64

All requests are queued at once (an offline batch), the engine admits, prefills and decodes them with continuous
batching, and one JSON line reports generated tokens per second, prompt tokens per second, mean time to first
token and the mean decode-step time. Greedy sampling on the device; the host reads one int per sequence per step.

Reference: the reference's serving figures are single-stream decode rates (docs/performance-notes.md:43-78); this is
the batched equivalent for the engine here.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    for name, default in (("layers", 32), ("dim", 4096), ("heads", 32), ("kv-heads", 8), ("ff", 14336), ("vocab", 128256),
                          ("requests", 256), ("prompt", 512), ("gen", 128), ("max-batch", 64), ("max-positions", 4096),
                          ("prefill-tokens", 8192)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--quant", choices=["none", "int8", "int4"], default="none")
    a = ap.parse_args(argv)
    from .. import _native
    from ..models import DecoderSpec, build_decoder
    from ..serve import GenerationOptions, LLMEngine
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    spec = DecoderSpec.llama(layers=a.layers, dim=a.dim, heads=a.heads, kv_heads=a.kv_heads, ff_dim=a.ff, vocab=a.vocab,
                             max_positions=a.max_positions)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = build_decoder(spec)
    torch.set_default_dtype(torch.float32)
    model = model.to(dev, torch.bfloat16).eval()
    if a.quant != "none":
        from ..quant import quantize_model
        quantize_model(model, a.quant)
    params = sum(p.numel() for p in model.parameters())
    blocks_needed = a.max_batch * ((a.prompt + a.gen + 15) // 16 + 1)
    eng = LLMEngine(model, num_blocks=blocks_needed + 64, max_batch=a.max_batch, max_prefill_tokens=a.prefill_tokens,
                    prefix_sharing=False, use_graph=not a.no_graph)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, a.vocab, (a.prompt,), generator=g).tolist() for _ in range(a.requests)]
    opts = GenerationOptions.greedy_options(a.gen)
    # warm-up: a few requests through both phases (kernel attributes, graphs for the steady batch size)
    eng.generate(prompts[: min(a.max_batch, a.requests)], GenerationOptions.greedy_options(4))
    torch.cuda.synchronize()
    steps0, gen0, pre0 = eng.steps, eng.tokens_generated, eng.tokens_prefilled
    for d in (eng.phase_seconds, eng.phase_steps):
        for k in d:
            d[k] = 0
    t0 = time.perf_counter()
    records = eng.generate(prompts, opts)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    _native.check_status("serve_bench")
    generated = eng.tokens_generated - gen0
    ttft = [r.first_token_at - r.arrival for r in records if r.first_token_at is not None]
    out = {"metric": "serving tokens/s (offline batch, greedy)", "value": round(generated / dt, 1), "unit": "tokens/s",
           "prompt_tokens_per_s": round((eng.tokens_prefilled - pre0) / dt, 1), "seconds": round(dt, 3),
           "requests": a.requests, "prompt": a.prompt, "gen": a.gen, "max_batch": a.max_batch,
           "steps": eng.steps - steps0, "ms_per_step": round(dt / max(eng.steps - steps0, 1) * 1e3, 3),
           "mean_ttft_s": round(sum(ttft) / max(len(ttft), 1), 3), "graph_replays": eng.runner.graph_replays,
           "parameters": params, "quant": a.quant, "dtype": "bf16",
           "model": f"llama-like {a.layers}L d{a.dim} h{a.heads}/{a.kv_heads} ff{a.ff} v{a.vocab}",
           "preemptions": eng.stats()["preemptions"],
           "prefill_seconds": round(eng.phase_seconds["prefill"], 3), "prefill_steps": eng.phase_steps["prefill"],
           "decode_seconds": round(eng.phase_seconds["decode"], 3), "decode_steps": eng.phase_steps["decode"],
           "ms_per_decode_step": round(eng.phase_seconds["decode"] / max(eng.phase_steps["decode"], 1) * 1e3, 3)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
