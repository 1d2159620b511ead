"""Device time of the serving collectives of a tensor-parallel group, one rank per GPU.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m idrak_b200.diag.tp_serve_collectives_bench

``all_reduce_rows`` (one-shot sum over the ranks' partial rows + residual add + RMS norm in one kernel, what follows the
row-parallel projections of a decode step) against ``dist.all_reduce`` + add + norm as three launches, for decode-sized
row counts; and the in-place two-shot all-reduce of the communicator against ``dist.all_reduce`` at prefill sizes. Every
figure is a CUDA-event time over a CUDA graph of many calls, the maximum over ranks, one JSON line per case on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time_graph(fn, calls: int, replays: int = 5) -> float:
    """ms per call of ``fn`` from a graph of ``calls`` calls."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(calls):
            fn()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / calls)
    t = torch.tensor([best], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--rows", type=int, nargs="*", default=[8, 64])
    ap.add_argument("--prefill-rows", type=int, nargs="*", default=[2048, 8192])
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from ..models.decoder import Norm
    from ..parallel.comm import Communicator
    from ..parallel.tp_serve import TPServeContext
    from .. import ops
    comm = Communicator(device=dev)
    tp = TPServeContext(comm, a.dim, max(a.rows), max(a.prefill_rows))
    norm = Norm(a.dim, "rms", 1e-5).to(dev, torch.bfloat16)
    for rows in a.rows:
        residual = torch.randn(rows, a.dim, device=dev).bfloat16()
        src = torch.randn(rows, a.dim, device=dev).bfloat16()

        def fused():
            tp.partial_buffer(rows).copy_(src)          # stands for the projection that writes its partial rows there
            tp.all_reduce_rows(tp.partial_buffer(rows), residual, norm)

        def copy_only():
            tp.partial_buffer(rows).copy_(src)

        scratch = torch.empty_like(src)

        def nccl():
            scratch.copy_(src)
            dist.all_reduce(scratch)
            x = ops.add(scratch, residual)
            norm(x)

        t_f, t_c, t_n = _time_graph(fused, 64), _time_graph(copy_only, 64), _time_graph(nccl, 64)
        if rank == 0:
            print(json.dumps({"case": "all_reduce_rows + residual + rms norm", "ranks": world, "rows": rows, "dim": a.dim,
                              "fused_us": round((t_f - t_c) * 1e3, 2), "nccl_add_norm_us": round((t_n - t_c) * 1e3, 2),
                              "copy_us": round(t_c * 1e3, 2)}), flush=True)
    for rows in a.prefill_rows:
        n = rows * a.dim
        buf = tp._bufs[0]
        view = buf.tensor(torch.bfloat16, n)
        view.normal_()
        mine = torch.randn(n, device=dev).bfloat16()

        def two_shot():
            comm.all_reduce(buf, torch.bfloat16, n)

        def nccl_big():
            dist.all_reduce(mine)

        t_f, t_n = _time_graph(two_shot, 8), _time_graph(nccl_big, 8)
        if rank == 0:
            gb = n * 2 / 1e9
            print(json.dumps({"case": "in-place all-reduce (prefill rows)", "ranks": world, "rows": rows, "dim": a.dim,
                              "mb": round(gb * 1e3, 1), "two_shot_us": round(t_f * 1e3, 1), "nccl_us": round(t_n * 1e3, 1),
                              "two_shot_bus_gbs": round(2 * (world - 1) / world * gb / (t_f * 1e-3), 1),
                              "nccl_bus_gbs": round(2 * (world - 1) / world * gb / (t_n * 1e-3), 1)}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    tp.close()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
