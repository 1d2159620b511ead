"""Worker run under torchrun by test_zero2.py: trains a small decoder with sharded gradients and writes the losses, the
final weights and what it held. argv: out path, steps. Not collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out, steps = sys.argv[1], int(sys.argv[2])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from zero3_worker import make_data, make_model
    from idrak_b200.parallel.zero2 import ShardedGradients
    model = make_model()
    total = sum(p.numel() for p in model.parameters())
    sharded = ShardedGradients(model, bucket_elems=20000)
    opt = torch.optim.AdamW(sharded.parameters(), lr=3e-3, weight_decay=0.0)
    data = make_data(steps)
    losses, held = [], 0
    for s in range(steps):
        b = data[s]
        mine = b[rank::world]
        loss = model.loss(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        loss.backward()
        sharded.finish_backward()
        assert all(p.grad is None for p in model.parameters()), "full gradients are released during backward"
        held = max(held, sharded.gradient_elems_held())
        opt.step()
        sharded.publish()
        opt.zero_grad()
        t = loss.detach().clone()
        dist.all_reduce(t)
        losses.append(float(t) / world)
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    if rank == 0:
        torch.save({"losses": losses, "state": {k: v.clone() for k, v in model.state_dict().items()}, "held": held,
                    "total": total, "peak_full": sharded.peak_full_gradient_elems, "buckets": len(sharded.buckets),
                    "same": all(torch.equal(parts[0], p) for p in parts)}, out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
