"""Link benchmark between the GPUs of a node: latency and bandwidth per ordered pair, cold and warm, and with all
pairs of a ring active at once.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29750 \
        -m idrak_b200.cluster.linkbench --bytes 268435456

Each measurement is a peer copy between symmetric buffers (device time, CUDA events, max over the two ranks).
Rank 0 prints one JSON line per pair and a summary. Reference: LinkBench (src/Idrak.Network/Bench/LinkBench.cs:63).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _copy_time(dst: torch.Tensor, src: torch.Tensor, iters: int) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        dst.copy_(src, non_blocking=True)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters / 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--small", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from ..parallel.comm import Communicator
    comm = Communicator(device=dev)
    buf = comm.symmetric(a.bytes)
    mine = buf.tensor(torch.uint8)
    src = torch.empty(a.bytes, dtype=torch.uint8, device=dev)
    from ..parallel.comm import _RawDeviceMemory
    results = []
    for shift in range(1, world):
        peer = (rank + shift) % world
        remote = torch.as_tensor(_RawDeviceMemory(buf.peer_ptrs[peer], a.bytes), device=dev)
        dist.barrier()
        cold = _copy_time(remote, src, 1)
        warm = _copy_time(remote, src, a.iters)
        lat = _copy_time(remote[: a.small], src[: a.small], 50)
        dist.barrier()
        row = torch.tensor([cold, warm, lat], device=dev, dtype=torch.float64)
        rows = [torch.empty_like(row) for _ in range(world)]
        dist.all_gather(rows, row)
        if rank == 0:
            for r, t in enumerate(rows):
                c, w, l = (float(x) for x in t)
                results.append({"from": r, "to": (r + shift) % world, "concurrent_pairs": world,
                                "cold_gbs": round(a.bytes / c / 1e9, 1), "warm_gbs": round(a.bytes / w / 1e9, 1),
                                "small_copy_us": round(l * 1e6, 2)})
    if rank == 0:
        for r in results:
            print(json.dumps(r))
        warm = [r["warm_gbs"] for r in results]
        print(json.dumps({"summary": True, "pairs": len(results), "warm_gbs_min": min(warm), "warm_gbs_max": max(warm),
                          "warm_gbs_mean": round(sum(warm) / len(warm), 1), "bytes": a.bytes}))
    dist.barrier()
    torch.cuda.synchronize()
    buf.close()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
