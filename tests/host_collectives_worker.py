"""Three gloo ranks run every host-collective algorithm; rank 0 writes the results."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch.distributed as dist

from idrak_b200.parallel.host_collectives import TorchTransport, create


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    v = torch.randn(5000, generator=torch.Generator().manual_seed(100 + rank))
    t = TorchTransport()
    out, same = {}, True
    for name, kw in (("naive", {}), ("ring", {}), ("hierarchical", {"nodes": [[0, 1], [2]]})):
        r = create(name, t, chunk=1024, **kw).all_reduce(v)
        out[name] = r
        parts = [torch.empty_like(r) for _ in range(3)]
        dist.all_gather(parts, r)
        same = same and all(torch.equal(p, parts[0]) for p in parts)
    c = create("ring", t)
    pieces = c.all_to_all([torch.full((4,), float(rank * 3 + j)) for j in range(3)])
    same = same and all(torch.equal(pieces[s], torch.full((4,), float(s * 3 + rank))) for s in range(3))
    if rank == 0:
        out["identical"] = same
        torch.save(out, sys.argv[1])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
