"""Worker run under torchrun by tests of pipeline / local-SGD / compression on gloo CPU ranks. Not collected.
argv: what ("pipeline" | "localsgd" | "compress"), out path, extra..."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _model(tie=False):
    from idrak_b200.models import DecoderSpec, build_decoder
    if tie:
        spec = DecoderSpec.gpt2(layers=4, dim=64, heads=4, vocab=300, max_positions=64)
    else:
        spec = DecoderSpec.llama(layers=4, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=300, max_positions=64)
    return build_decoder(spec, seed=9).float()


def _data(steps, batch=8, seq=32):
    g = torch.Generator().manual_seed(21)
    return torch.randint(0, 300, (steps, batch, seq + 1), generator=g)


def pipeline(out, stages, schedule, tie):
    from idrak_b200.parallel.pipeline import PipelineTrainer
    rank, world = dist.get_rank(), dist.get_world_size()
    tr = PipelineTrainer(_model(tie == "tie"), int(stages), micro_batches=4, schedule=schedule, lr=1e-3)
    replicas = world // int(stages)
    data = _data(3, batch=8 * replicas)
    losses = []
    for s in range(3):
        b = data[s][tr.layout.replica * 8:(tr.layout.replica + 1) * 8]
        losses.append(tr.train_step(b[:, :-1], b[:, 1:]))
    states = [None] * world
    dist.all_gather_object(states, (tr.layout.stage, tr.layout.replica, tr.stage_state()))
    if rank == 0:
        torch.save({"losses": losses, "states": states}, out)


def localsgd(out, every, momentum):
    from idrak_b200.ops import FusedAdamW
    from idrak_b200.parallel.local_sgd import LocalSGD
    rank, world = dist.get_rank(), dist.get_world_size()
    model = _model()
    opt = FusedAdamW(model.decay_groups(0.0), lr=1e-3, weight_decay=0.0)
    ls = LocalSGD(model.parameters(), opt, sync_every=int(every), outer_momentum=float(momentum))
    data = _data(8, batch=4 * world)
    spread = []
    for s in range(8):
        b = data[s][rank * 4:(rank + 1) * 4]
        opt.zero_grad()
        model.loss(b[:, :-1].int(), b[:, 1:].int()).backward()
        synced = ls.step()
        flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        parts = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(parts, flat)
        spread.append((bool(synced), float((parts[0] - parts[-1]).abs().max())))
    if rank == 0:
        with open(out, "w") as f:
            json.dump({"spread": spread, "syncs": ls.syncs}, f)


def compress(out, kind):
    from idrak_b200.parallel.compression import CompressedGradientReducer
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(5 + rank)
    params = [torch.nn.Parameter(torch.zeros(3000)), torch.nn.Parameter(torch.zeros(50, 70))]
    red = CompressedGradientReducer(params, kind=kind, bucket_elems=2048, top_k=0.1)
    sent_total = [torch.zeros_like(p) for p in params]
    true_total = [torch.zeros_like(p) for p in params]
    for step in range(6):
        grads = [torch.randn_like(p) for p in params]
        for p, g in zip(params, grads):
            p.grad = g.clone()
        for t, g in zip(true_total, grads):
            gs = [torch.empty_like(g) for _ in range(world)]
            dist.all_gather(gs, g)
            t += sum(gs) / world
        red.reduce()
        for t, p in zip(sent_total, params):
            t += p.grad
    same = []
    for p in params:
        gs = [torch.empty_like(p.grad) for _ in range(world)]
        dist.all_gather(gs, p.grad)
        same.append(bool(all(torch.equal(gs[0], g) for g in gs)))
    err = max(float((a - b).abs().max()) for a, b in zip(sent_total, true_total))
    one = max(float((p.grad - 0).abs().max()) for p in params)
    if rank == 0:
        with open(out, "w") as f:
            json.dump({"identical_on_ranks": all(same), "accumulated_error": err, "ratio": red.compressor.ratio(),
                       "last_max": one}, f)


def main():
    dist.init_process_group("gloo")
    what, out, rest = sys.argv[1], sys.argv[2], sys.argv[3:]
    {"pipeline": pipeline, "localsgd": localsgd, "compress": compress}[what](out, *rest)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
