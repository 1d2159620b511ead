"""LoRA fine-tuning throughput over a frozen quantised base: a Llama-8B-shaped decoder with random weights packed to
int4 (symmetric, groups of 32, fp16 scales) or int8, rank-16 adapters on q / k / v / o / gate / up / down, bf16
activations, uniform random tokens. One process per GPU; with several GPUs the adapter gradients go through the fused
data-parallel path (reduce-scatter + AdamW shard update + all-gather in one kernel per bucket).

    python -m idrak_b200.diag.lora_bench --base int4 --seq 2048 --micro-batch 4 --steps 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29720 \
        -m idrak_b200.diag.lora_bench --base int4

Rank 0 prints one JSON line: tokens per second over all ranks (CUDA events, max over ranks), milliseconds per step,
peak memory.

Reference: FineTuner.Train over an int4 / int8 base (src/Idrak.Text/FineTuning.cs:1176; defaults rank 16, alpha 32,
targets q, k, v, o, gate, up, down).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    for name, default in (("layers", 32), ("dim", 4096), ("heads", 32), ("kv-heads", 8), ("ff", 14336), ("vocab", 128256),
                          ("seq", 2048), ("micro-batch", 4), ("steps", 5), ("warmup", 3), ("rank", 16)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--base", choices=["bf16", "int8", "int4", "fp8"], default="int4")
    ap.add_argument("--checkpoint-blocks", action="store_true")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    from .. import _native
    from ..adapters.lora import add_adapters
    from ..models import DecoderSpec, build_decoder
    from ..ops import FusedAdamW
    from ..quant import quantize_model

    spec = DecoderSpec.llama(layers=a.layers, dim=a.dim, heads=a.heads, kv_heads=a.kv_heads, ff_dim=a.ff, vocab=a.vocab,
                             max_positions=a.seq)
    torch.set_default_dtype(torch.bfloat16)
    torch.manual_seed(1234)                                 # the same base on every rank
    torch.cuda.manual_seed(1234)
    with torch.device(dev):
        model = build_decoder(spec)
    torch.set_default_dtype(torch.float32)
    model = model.to(dev, torch.bfloat16)
    if a.base != "bf16":
        quantize_model(model, a.base)
        torch.cuda.empty_cache()
    trainable = add_adapters(model, rank=a.rank, alpha=2.0 * a.rank)
    model.checkpoint_blocks = bool(a.checkpoint_blocks)
    model.train()
    if world > 1:
        from ..parallel.dp import DataParallel
        sync = DataParallel(model, lr=2e-4, betas=(0.9, 0.999), weight_decay=0.0, max_grad_norm=1.0)
        opt = sync.optimizer
    else:
        sync = None
        opt = FusedAdamW(trainable, lr=2e-4, betas=(0.9, 0.999), weight_decay=0.0, max_grad_norm=1.0)
    gen = torch.Generator().manual_seed(1000 + rank)
    batches = [torch.randint(0, a.vocab, (a.micro_batch, a.seq + 1), generator=gen, dtype=torch.int32).to(dev) for _ in range(4)]

    from ..training import TrainStep
    runner = TrainStep(model, opt, sync=sync, use_graph=False, ignore_index=None)
    pairs = [(b[:, :-1].contiguous(), b[:, 1:].contiguous()) for b in batches]

    def step(i):
        ids, tgt = pairs[i % len(pairs)]
        return runner(ids, tgt)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(a.warmup, 1)):
        loss = step(i)
    barrier()
    _native.check_status("lora_bench warm-up")
    torch.cuda.reset_peak_memory_stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    e1.record()
    barrier()
    _native.check_status("lora_bench")
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        per_step = float(ms) / a.steps
        tokens = a.micro_batch * a.seq * world
        n_train = sum(p.numel() for p in trainable)
        print(json.dumps({"metric": "LoRA fine-tune tokens/s", "value": round(tokens / (per_step / 1e3), 1), "unit": "tokens/s",
                          "n_gpus": world, "ms_per_step": round(per_step, 2), "peak_memory_gib": round(float(peak), 1),
                          "trainable_parameters": n_train, "final_loss": round(float(loss.item()), 4), "steps": a.steps,
                          "warmup": a.warmup, "dtype": "bf16 activations", "data": "uniform random tokens, random-init weights",
                          "config": {"model": f"llama-like {a.layers}L d{a.dim} h{a.heads}/{a.kv_heads} ff{a.ff} v{a.vocab}",
                                     "base": a.base, "rank": a.rank, "alpha": 2.0 * a.rank, "seq_len": a.seq,
                                     "micro_batch": a.micro_batch, "parallelism": f"dp{world}",
                                     "checkpoint_blocks": bool(a.checkpoint_blocks)}}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
