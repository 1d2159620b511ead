"""Worker for the rollout exchange test (run under torchrun, gloo). argv: out path. Not collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def episodes_of(rank):
    g = torch.Generator().manual_seed(rank)
    return [torch.randint(0, 100, (int(n),), generator=g) for n in torch.randint(1, 9, (rank + 1,), generator=g)]


def main():
    dist.init_process_group("gloo")
    from idrak_b200.rl import exchange_rollouts
    rank = dist.get_rank()
    got = exchange_rollouts(episodes_of(rank))
    empty = exchange_rollouts([] if rank == 0 else [torch.tensor([1.5, 2.5])])
    if rank == 0:
        torch.save({"all": got, "empty": empty}, sys.argv[1])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
