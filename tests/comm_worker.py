"""Rank process of the communicator test: every peer-memory collective against its NCCL twin, and two gathers in a
row into one buffer while one rank is slow to read the first result."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from idrak_b200 import _native
    from idrak_b200.parallel.comm import Communicator
    comm = Communicator(device=dev)
    ok = {}
    n = world * 8 * 1024
    g = torch.Generator(device=dev).manual_seed(11 + rank)

    # all-reduce (two-shot), bf16 and fp32
    for dtype in (torch.bfloat16, torch.float32):
        buf = comm.symmetric(n * 4)
        t = buf.tensor(dtype, n)
        t.copy_(torch.randn(n, generator=g, device=dev).to(dtype))
        ref = t.float().clone()
        dist.all_reduce(ref)
        got = comm.all_reduce(buf, dtype, n).float()
        ok[f"all_reduce_{dtype}"] = bool((got - ref).abs().max() <= (0.05 if dtype == torch.bfloat16 else 1e-4))
        parts = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(parts, got)
        ok[f"all_reduce_same_bits_{dtype}"] = all(torch.equal(p, parts[0]) for p in parts)
        torch.cuda.synchronize()
        dist.barrier()
        buf.close()

    # reduce-scatter
    buf = comm.symmetric(n * 2)
    t = buf.tensor(torch.bfloat16, n)
    t.copy_(torch.randn(n, generator=g, device=dev).to(torch.bfloat16))
    full = t.float().clone()
    dist.all_reduce(full)
    out = torch.empty(n // world, dtype=torch.float32, device=dev)
    comm.reduce_scatter(buf, torch.bfloat16, n, out)
    ok["reduce_scatter"] = bool((out - full[rank * (n // world):(rank + 1) * (n // world)]).abs().max() < 1e-3)
    torch.cuda.synchronize()
    dist.barrier()

    # two gathers in a row into one buffer; the last rank is slow to consume the first result
    sl = n // world
    first = torch.full((sl,), float(rank + 1), dtype=torch.bfloat16, device=dev)
    second = torch.full((sl,), float(10 * (rank + 1)), dtype=torch.bfloat16, device=dev)
    g1 = comm.all_gather(buf, first)
    if rank == world - 1:
        torch.cuda._sleep(200_000_000)                 # ~0.1 s on the stream, before this rank reads gather one
    seen_first = g1.clone()                            # stream-ordered consumer of the first result
    g2 = comm.all_gather(buf, second)
    seen_second = g2.clone()
    torch.cuda.synchronize()
    want1 = torch.cat([torch.full((sl,), float(r + 1)) for r in range(world)])
    want2 = torch.cat([torch.full((sl,), float(10 * (r + 1))) for r in range(world)])
    ok["gather_first_intact"] = bool(torch.equal(seen_first.float().cpu(), want1))
    ok["gather_second"] = bool(torch.equal(seen_second.float().cpu(), want2))

    # broadcast twice, a slow receiver in between
    raw = buf.tensor(torch.float32, 4096)
    raw.fill_(float(rank))
    torch.cuda.synchronize()
    dist.barrier()
    comm.broadcast(buf, 4096 * 4, root=0)
    if rank == world - 1:
        torch.cuda._sleep(100_000_000)
    b1 = raw.clone()
    if rank == 0:
        raw.fill_(7.0)
    comm.broadcast(buf, 4096 * 4, root=0)
    b2 = raw.clone()
    torch.cuda.synchronize()
    ok["broadcast_first"] = bool((b1 == 0).all())
    ok["broadcast_second"] = bool((b2 == 7).all())

    small = comm.all_reduce_small(torch.tensor([1.0 + rank, 2.0], device=dev))
    ok["small"] = bool(small[0].item() == sum(1.0 + r for r in range(world)) and small[1].item() == 2.0 * world)
    torch.cuda.synchronize()
    _native.check_status("comm worker")
    # guard bands: intact after every collective above; a write one byte past the end of a buffer is noticed
    comm.check_canaries()
    ok["canaries_intact"] = True
    probe = comm.symmetric(1024, "probe")
    probe._whole[probe.GUARD + probe.nbytes] = 0              # what an overrunning kernel would do
    try:
        comm.check_canaries()
        ok["canary_trips"] = False
    except RuntimeError as e:
        ok["canary_trips"] = "probe" in str(e)
    probe.close()
    rows = comm.network_summary(gather=True)
    mine = rows[rank]["collectives"]
    ok["summary_rows"] = len(rows) == world and rows[rank]["rank"] == rank
    ok["summary_counts"] = (mine["all_reduce"]["calls"] == 2 and mine["all_gather"]["calls"] == 2
                            and mine["all_gather"]["bytes_sent"] == 2 * (world - 1) * sl * 2
                            and mine["reduce_scatter"]["bytes_read"] == (world - 1) * n * 2 // world)
    gathered = [None] * world
    dist.all_gather_object(gathered, ok)
    if rank == 0:
        torch.save(gathered, out_path)
    dist.barrier()
    buf.close()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
