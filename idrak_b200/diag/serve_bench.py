"""Serving throughput of the continuous-batching engine with random weights of a given architecture, on one GPU or
tensor-parallel over the ranks of a torchrun launch.

    python -m idrak_b200.diag.serve_bench --layers 32 --dim 4096 --heads 32 --kv-heads 8 --ff 14336 \
        --vocab 128256 --requests 256 --prompt 512 --gen 128 --max-batch 64
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m idrak_b200.diag.serve_bench \
        --tp 8 --requests 64 --prompt-min 128 --prompt-max 2048 --gen 256 --max-batch 64 [--quant int8] [--arm nccl]

With ``--tp N`` every rank builds its slice of the model (``parallel.tp_serve.random_shard``) and runs the engine in
lock-step over the same requests; ``--arm nccl`` swaps the fused peer-memory all-reduce for ``dist.all_reduce`` and
this library's GEMMs for cuBLAS (``torch.nn.functional.linear``) - the baseline the fused path is measured against.
Times are device times (CUDA events), maximum over ranks.

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
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (run under torchrun with as many processes)")
    ap.add_argument("--prompt-min", type=int, default=0, help="with --prompt-max: prompt lengths uniform in [min, max]")
    ap.add_argument("--prompt-max", type=int, default=0)
    ap.add_argument("--arm", choices=["fused", "nccl"], default="fused")
    ap.add_argument("--fold-norms", action="store_true", help="fold the RMS norm weights into the projections (one GPU)")
    ap.add_argument("--kv", choices=["bf16", "int8"], default="bf16", help="key / value cache element type")
    a = ap.parse_args(argv)
    import os
    from .. import _native
    from ..models import DecoderSpec, build_decoder
    from ..serve import GenerationOptions, LLMEngine
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.tp > 1 and world != a.tp:
        raise SystemExit(f"--tp {a.tp} needs {a.tp} ranks (torchrun --nproc-per-node {a.tp}); this launch has {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    spec = DecoderSpec.llama(layers=a.layers, dim=a.dim, heads=a.heads, kv_heads=a.kv_heads, ff_dim=a.ff, vocab=a.vocab,
                             max_positions=a.max_positions)
    tp = None
    if a.tp > 1:
        import torch.distributed as dist
        from ..parallel.comm import Communicator
        from ..parallel.tp_serve import TPServeContext, random_shard
        dist.init_process_group("nccl", device_id=dev)
        model = random_shard(spec, rank, world, dev)
        comm = Communicator(device=dev)
        tp = TPServeContext(comm, spec.dim, max_rows=256, max_prefill_rows=a.prefill_tokens + 64)
    else:
        torch.set_default_dtype(torch.bfloat16)
        with torch.device(dev):
            model = build_decoder(spec)
        torch.set_default_dtype(torch.float32)
        model = model.to(dev, torch.bfloat16).eval()
    if a.quant != "none":
        from ..quant import quantize_model
        quantize_model(model, a.quant)
    params = sum(p.numel() for p in model.parameters()) * (world if tp is not None else 1)
    longest = a.prompt_max if a.prompt_max > 0 else a.prompt
    blocks_needed = a.max_batch * ((longest + a.gen + 15) // 16 + 1)
    eng = LLMEngine(model, num_blocks=blocks_needed + 64, max_batch=a.max_batch, max_prefill_tokens=a.prefill_tokens,
                    prefix_sharing=False, use_graph=not a.no_graph, tp=tp, fold_norms=a.fold_norms,
                    kv_dtype=torch.int8 if a.kv == "int8" else None)
    if tp is not None and a.arm == "nccl":
        _use_nccl_arm(eng.runner)
    g = torch.Generator().manual_seed(0)
    if a.prompt_max > 0:
        lengths = torch.randint(max(a.prompt_min, 1), a.prompt_max + 1, (a.requests,), generator=g).tolist()
    else:
        lengths = [a.prompt] * a.requests
    prompts = [torch.randint(0, a.vocab, (n,), generator=g).tolist() for n in lengths]
    opts = GenerationOptions.greedy_options(a.gen)
    # warm-up: a few requests through both phases (kernel attributes, graphs for the steady batch size)
    eng.generate(prompts[: min(a.max_batch, a.requests)], GenerationOptions.greedy_options(4))
    torch.cuda.synchronize()
    steps0, gen0, pre0 = eng.steps, eng.tokens_generated, eng.tokens_prefilled
    for d in (eng.phase_seconds, eng.phase_steps):
        for k in d:
            d[k] = 0
    if tp is not None:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    records = eng.generate(prompts, opts)
    e1.record()
    torch.cuda.synchronize()
    dt = max(time.perf_counter() - t0, e0.elapsed_time(e1) / 1e3)
    _native.check_status("serve_bench")
    generated = eng.tokens_generated - gen0
    ttft = sorted(r.first_token_at - r.arrival for r in records if r.first_token_at is not None)
    if tp is not None:
        # the slowest rank sets the time
        t = torch.tensor([dt, eng.phase_seconds["prefill"], eng.phase_seconds["decode"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt, eng.phase_seconds["prefill"], eng.phase_seconds["decode"] = (float(v) for v in t)
    out = {"metric": "serving tokens/s (offline batch, greedy)", "value": round(generated / dt, 1), "unit": "tokens/s",
           "prompt_tokens_per_s": round((eng.tokens_prefilled - pre0) / dt, 1), "seconds": round(dt, 3),
           "requests": a.requests, "prompt": a.prompt, "gen": a.gen, "max_batch": a.max_batch,
           "steps": eng.steps - steps0, "ms_per_step": round(dt / max(eng.steps - steps0, 1) * 1e3, 3),
           "mean_ttft_s": round(sum(ttft) / max(len(ttft), 1), 3),
           "p50_ttft_s": round(ttft[len(ttft) // 2], 3) if ttft else None,
           "prefill_tokens_per_s": round((eng.tokens_prefilled - pre0) / max(eng.phase_seconds["prefill"], 1e-9), 1),
           "decode_tokens_per_s": round((generated - eng.phase_steps["prefill"]) / max(eng.phase_seconds["decode"], 1e-9), 1)
           if eng.phase_steps["decode"] else None,
           "tp": a.tp, "arm": a.arm if a.tp > 1 else None, "n_gpus": world,
           "prompt_lengths": ([a.prompt_min, a.prompt_max] if a.prompt_max > 0 else a.prompt),
           "graph_replays": eng.runner.graph_replays,
           "parameters": params, "quant": a.quant, "dtype": "bf16",
           "model": f"llama-like {a.layers}L d{a.dim} h{a.heads}/{a.kv_heads} ff{a.ff} v{a.vocab}",
           "preemptions": eng.stats()["preemptions"],
           "prefill_seconds": round(eng.phase_seconds["prefill"], 3), "prefill_steps": eng.phase_steps["prefill"],
           "decode_seconds": round(eng.phase_seconds["decode"], 3), "decode_steps": eng.phase_steps["decode"],
           "ms_per_decode_step": round(eng.phase_seconds["decode"] / max(eng.phase_steps["decode"], 1) * 1e3, 3)}
    if rank == 0:
        print(json.dumps(out))
    if tp is not None:
        tp.close()
        comm.close()
        dist.destroy_process_group()
    return 0


def _use_nccl_arm(runner) -> None:
    """The comparison arm of a tensor-parallel run: NCCL for the sum over ranks, cuBLAS for the products."""
    import torch.distributed as dist
    from .. import ops

    def sum_partials(partial, residual, norm=None):
        total = partial.contiguous()
        dist.all_reduce(total)
        x = total + residual
        return x, (norm(x) if norm is not None else None)

    runner._sum_partials = sum_partials
    ops.linear = lambda x, w, b=None, residual=None: (
        torch.nn.functional.linear(x, w, b) + (residual if residual is not None else 0))
    import idrak_b200.ops.gemm as g
    g.linear = ops.linear
    import idrak_b200.models.decoder as d
    d.ops.linear = ops.linear


if __name__ == "__main__":
    raise SystemExit(main())
