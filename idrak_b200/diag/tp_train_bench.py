"""Training-step throughput of a tensor-parallel decoder (Llama-8B shape by default) with random weights and uniform
random tokens: forward, backward and the AdamW step of the sliced model, every rank seeing the whole batch
(sequence-parallel activations between blocks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29710 \
        -m idrak_b200.diag.tp_train_bench --mode fused --steps 5 --warmup 3

``--mode fused`` runs the all-gather -> GEMM and GEMM -> reduce-scatter kernels of ``csrc/tp_gemm.cu``; ``--mode nccl``
runs NCCL collectives followed by the same GEMMs (the baseline). Rank 0 prints one JSON line: tokens per second over
all ranks (CUDA events around the timed steps, max over ranks), milliseconds per step, model FLOPs per second.

Reference: the reference has no tensor parallelism (its 8 B-class runs use ZeRO or pipeline placement); this is the
measurement for the tensor-parallel training configuration.
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
                          ("seq", 4096), ("batch", 8), ("steps", 5), ("warmup", 3)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--mode", choices=["fused", "nccl"], default="fused")
    ap.add_argument("--checkpoint-blocks", action="store_true")
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from .. import _native
    from ..models import DecoderSpec
    from ..parallel.tp import TensorParallel
    from ..parallel.tp_layers import TPDecoder, TPOptimizer

    spec = DecoderSpec.llama(layers=a.layers, dim=a.dim, heads=a.heads, kv_heads=a.kv_heads, ff_dim=a.ff, vocab=a.vocab,
                             max_positions=a.seq, theta=500000.0, eps=1e-5)
    tokens = a.batch * a.seq
    if a.mode == "fused":
        from ..parallel.comm import Communicator
        tp = TensorParallel(Communicator(device=dev), max_rows=tokens, max_in=a.dim, max_out=a.dim)
    else:
        tp = TensorParallel(mode="nccl")
    model = TPDecoder(spec, tp).to(dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02, generator=g)
            else:
                p.fill_(1.0)
    if a.checkpoint_blocks and not hasattr(model, "checkpoint_blocks"):
        raise SystemExit("this build's tensor-parallel decoder keeps its activations; --checkpoint-blocks is not available")
    if a.checkpoint_blocks:
        model.checkpoint_blocks = True
    opt = TPOptimizer(model, lr=3e-4, weight_decay=0.1, max_grad_norm=1.0, betas=(0.9, 0.95))
    data_gen = torch.Generator().manual_seed(99)           # the same batch on every rank
    batches = [torch.randint(0, a.vocab, (a.batch, a.seq + 1), generator=data_gen, dtype=torch.int32).to(dev) for _ in range(4)]

    def step(i):
        b = batches[i % len(batches)]
        opt.zero_grad()
        loss = model.loss(b[:, :-1].contiguous(), b[:, 1:].contiguous())
        loss.backward()
        opt.step()
        return loss

    for i in range(max(a.warmup, 1)):
        loss = step(i)
    torch.cuda.synchronize()
    dist.barrier()
    _native.check_status("tp_train_bench warm-up")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    _native.check_status("tp_train_bench")
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device=dev, dtype=torch.float64)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        per_step = float(ms) / a.steps
        params = a.layers * (a.dim * (a.heads + 2 * a.kv_heads) * (a.dim // a.heads) + a.dim * a.dim + 3 * a.dim * a.ff) + a.vocab * a.dim
        attn = a.layers * 2 * 2 * a.seq * a.dim * 0.5              # causal scores + values per token, forward
        flops = 3 * tokens * (2 * params + attn)                   # forward + backward
        print(json.dumps({"metric": "train tokens/s (tensor parallel)", "value": round(tokens / (per_step / 1e3), 1),
                          "unit": "tokens/s", "n_gpus": world, "mode": a.mode, "ms_per_step": round(per_step, 2),
                          "model_tflops_per_gpu": round(flops / (per_step / 1e3) / 1e12 / world, 1),
                          "peak_memory_gib": round(float(peak), 1), "final_loss": round(float(loss.item()), 4),
                          "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "uniform random tokens, random-init weights",
                          "config": {"model": f"llama-like {a.layers}L d{a.dim} h{a.heads}/{a.kv_heads} ff{a.ff} v{a.vocab}",
                                     "seq_len": a.seq, "global_batch": a.batch, "parallelism": f"tp{world}",
                                     "checkpoint_blocks": bool(a.checkpoint_blocks)}}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
