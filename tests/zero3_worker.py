"""Worker run under torchrun by test_zero3.py: trains a small decoder with its blocks' parameters sharded over the
ranks and writes the losses and the gathered final weights. argv: out path, steps. Not collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_model():
    from idrak_b200.models import DecoderSpec, build_decoder
    return build_decoder(DecoderSpec.llama(layers=3, dim=48, heads=4, kv_heads=2, ff_dim=96, vocab=128, max_positions=32), seed=5)


def make_data(steps, batch=8, seq=24):
    return torch.randint(0, 128, (steps, batch, seq + 1), generator=torch.Generator().manual_seed(9))


def main():
    out, steps = sys.argv[1], int(sys.argv[2])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200.parallel.zero3 import ShardedParameters
    model = make_model()
    total = sum(p.numel() for p in model.parameters())
    sharded = ShardedParameters(model, units=list(model.blocks))
    held = sum(p.numel() for p in sharded.parameters())
    assert sharded.gathered_bytes() == 0                       # nothing gathered at rest
    opt = torch.optim.AdamW(sharded.parameters(), lr=3e-3, weight_decay=0.0)
    data = make_data(steps)
    losses = []
    for s in range(steps):
        b = data[s]
        mine = b[rank::world]                                   # each rank its slice of the global batch
        loss = model.loss(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        loss.backward()
        sharded.finish_backward()
        assert sharded.gathered_bytes() == 0
        opt.step()
        opt.zero_grad()
        t = loss.detach().clone()
        dist.all_reduce(t)
        losses.append(float(t) / world)
    state = sharded.full_state()
    if rank == 0:
        torch.save({"losses": losses, "state": state, "held": held, "total": total}, out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
