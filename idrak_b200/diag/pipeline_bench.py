"""Pipeline-parallel training step on GPUs: tokens/s of GPipe and 1F1B over ``stages x replicas`` ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \\
        -m idrak_b200.diag.pipeline_bench --stages 4 --micro-batches 8 --schedule 1f1b

Activations and their gradients cross the stage boundaries by NCCL point-to-point sends (NVLink); every stage runs
this library's kernels for its layers and its own fused AdamW. Timed with CUDA events after warm-up, maximum over
ranks; rank 0 prints one JSON line with the measured step, the ideal bubble of the schedule and the efficiency against
``stages`` times the one-stage rate when ``--baseline`` is given.

Reference: PipelinePretraining (src/Idrak.Text/PipelinePretraining.cs), GPipeSchedule
(src/Idrak.Network/Training/PipelineSchedules.cs:6-40).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    for name, default in (("layers", 12), ("dim", 768), ("heads", 12), ("vocab", 50304), ("seq", 1024), ("batch", 16),
                          ("stages", 2), ("micro-batches", 8), ("steps", 10), ("warmup", 3)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--schedule", choices=["gpipe", "1f1b"], default="1f1b")
    ap.add_argument("--baseline", type=float, default=0.0, help="tokens/s of the same model on one GPU, for the efficiency")
    a = ap.parse_args(argv)
    from .. import _native
    from ..models import DecoderSpec, build_decoder
    from ..parallel.pipeline import PipelineTrainer, ideal_bubble
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if world % a.stages:
        raise SystemExit(f"{world} ranks do not divide into {a.stages} stages")
    replicas = world // a.stages
    spec = DecoderSpec.gpt2(layers=a.layers, dim=a.dim, heads=a.heads, vocab=a.vocab, max_positions=a.seq)
    model = build_decoder(spec, seed=1).to(dev, torch.bfloat16)
    trainer = PipelineTrainer(model, a.stages, a.micro_batches, a.schedule, lr=3e-4)
    del model
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(7 + rank // a.stages)           # one stream of batches per replica
    batches = [torch.randint(0, a.vocab, (a.batch, a.seq + 1), generator=g) for _ in range(4)]

    def step(i):
        b = batches[i % len(batches)]
        return trainer.train_step(b[:, :-1].contiguous(), b[:, 1:].contiguous())
    for i in range(a.warmup):
        loss = step(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = _native.lib().idrak_launch_count()
    e0.record()
    for i in range(a.steps):
        loss = step(a.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    _native.check_status("pipeline bench")
    tokens = a.batch * a.seq * replicas
    if rank == 0:
        rate = tokens / (float(ms) / 1e3)
        out = {"metric": "pipeline-parallel train tokens/s", "value": round(rate, 1), "unit": "tokens/s",
               "ms_per_step": round(float(ms), 3), "n_gpus": world, "stages": a.stages, "replicas": replicas,
               "micro_batches": a.micro_batches, "schedule": a.schedule,
               "ideal_bubble": round(ideal_bubble(a.stages, a.micro_batches), 4), "final_loss": round(float(loss), 4),
               "kernels_of_this_library_per_step_on_rank0": (_native.lib().idrak_launch_count() - before) // a.steps,
               "model": f"gpt2-like {a.layers}L d{a.dim}", "batch_per_replica": a.batch, "seq": a.seq,
               "memory_gib_rank0": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)}
        if a.baseline > 0:
            out["efficiency_vs_gpus_x_one_gpu"] = round(rate / (a.baseline * world), 3)
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
