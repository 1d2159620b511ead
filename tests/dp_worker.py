"""Worker run under torchrun by the multi-GPU tests: trains a small decoder for a few steps data-parallel and
writes what rank 0 ends with, so the launcher can compare modes. Not collected by pytest."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode, out_path, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200 import _native
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.parallel.dp import DataParallel
    from idrak_b200.training import TrainStep

    spec = DecoderSpec.gpt2(layers=2, dim=256, heads=4, vocab=1000, max_positions=128)
    model = build_decoder(spec, seed=7).to(dev, torch.bfloat16)
    uneven = mode.endswith("_header")         # ranks hold different numbers of sequences; the header carries the weights
    mode = mode.replace("_header", "")
    sync = DataParallel(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, mode=mode, bucket_mb=0.5)
    step = TrainStep(model, sync.optimizer, sync=sync, use_graph=False, ignore_index=None)
    g = torch.Generator().manual_seed(100)
    data = torch.randint(0, 1000, (steps, world * 4, 129), generator=g)
    losses = []
    total = world * 4
    cuts = [0] + [2 + 4 * r for r in range(world - 1)] + [total] if uneven else [4 * r for r in range(world + 1)]
    headers = []
    for s in range(steps):
        mine = data[s, cuts[rank]:cuts[rank + 1]].to(dev)
        if uneven:
            h = sync.step_header(mine.shape[0] * 128, stop=(s == steps - 1 and rank == world - 1))
            headers.append((float(h["tokens"]), float(h["stop"])))
        loss = step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        losses.append(float(loss.item()))
    torch.cuda.synchronize()
    _native.check_status("dp_worker")
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    # every rank must hold identical weights
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    same = all(torch.equal(gathered[0], t) for t in gathered)
    if rank == 0:
        torch.save({"weights": flat.cpu(), "losses": losses, "same": same, "grad_norm": sync.optimizer.grad_norm(),
                    "headers": headers}, out_path)
    sync.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
