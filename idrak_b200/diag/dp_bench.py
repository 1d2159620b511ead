"""Device time of the fused data-parallel kernels on one bucket, against their roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m idrak_b200.diag.dp_bench \\
        --bucket-mb 64 [--blocks 32] [--update-blocks 296]

Every rank owns a symmetric gradient bucket and parameter bucket of ``--bucket-mb`` MiB of bf16. Timed with CUDA
events after warm-up, maximum over ranks:

* ``dp_reduce_scatter``: a rank reads its 1/W slice from all W ranks (W - 1 of them over NVLink), sums in rank
  order, writes the fp32 shard gradient. NVLink bytes in per rank: (W-1)/W x bucket bytes; HBM bytes: slice read
  plus 2 x slice written as fp32.
* ``dp_adamw_allgather``: AdamW on the fp32 shard (gradient, master, two moments read; master and moments written:
  28 B per parameter of the shard) and the new bf16 weights stored into all W parameter buffers (W - 1 over NVLink).

The roofline time of each is the larger of HBM bytes / measured copy bandwidth and NVLink bytes / measured peer
bandwidth per direction; the JSON line gives the achieved fraction. One line per kernel, printed by rank 0.

Reference: the reduction these kernels replace runs on the CPU over host-staged buckets
(src/Idrak.Network/Training/GradientReduction.cs:625-640, Sharding.cs:229-338).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bucket-mb", type=float, default=64.0)
    ap.add_argument("--blocks", type=int, default=32, help="CTAs of the reduce-scatter (it shares the SMs with backward)")
    ap.add_argument("--update-blocks", type=int, default=0, help="CTAs of the update + all-gather (0: two per SM)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=0.0, help="measured copy bandwidth (default: MEASURED_PEAKS.json or 6650)")
    ap.add_argument("--nvlink-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    a = ap.parse_args(argv)
    from .. import _native
    from ..ops.optim import H_B1, H_B2, H_BC1, H_BC2, H_CLIP, H_COUNT, H_EPS, H_GSCALE, H_LR, H_MAXNORM
    from ..parallel.comm import CH_BUCKET0, CH_STEP_DONE, Communicator
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    hbm = a.hbm_gbs
    if hbm <= 0:
        hbm = 6650.0
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        try:
            hbm = float(json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))["hbm_gbs"])
        except Exception:
            pass
    lib = _native.lib()
    comm = Communicator(device=dev)
    n = int(a.bucket_mb * 1024 * 1024 / 2) // (world * 1024) * (world * 1024)
    grads = comm.symmetric(n * 2)
    params = comm.symmetric(n * 2)
    grads.tensor(torch.bfloat16, n).normal_()
    params.tensor(torch.bfloat16, n).normal_()
    sl = n // world
    shard_grad = torch.zeros(sl, dtype=torch.float32, device=dev)
    master = torch.randn(sl, dtype=torch.float32, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    partial = torch.zeros(max(a.blocks, 1), dtype=torch.float32, device=dev)
    flags = torch.ones(n // 128 + 1, dtype=torch.uint8, device=dev)
    hyper = torch.zeros(H_COUNT, dtype=torch.float32, device=dev)
    for k, val in ((H_LR, 1e-4), (H_B1, 0.9), (H_B2, 0.95), (H_EPS, 1e-8), (H_BC1, 0.1), (H_BC2, 0.05), (H_CLIP, 1.0),
                   (H_MAXNORM, 1.0), (H_GSCALE, 1.0)):
        hyper[k] = val
    ub = a.update_blocks or 2 * lib.idrak_sm_count()
    stream = torch.cuda.current_stream().cuda_stream

    def reduce_scatter():
        comm.bump_epoch()
        _native.check(lib.idrak_dp_reduce_scatter(comm.ctx, grads.ptr_array, 0, n, 0, shard_grad.data_ptr(),
                                                  partial.data_ptr(), None, CH_BUCKET0, a.blocks, stream), "rs")

    def update():
        comm.bump_epoch()
        _native.check(lib.idrak_dp_adamw_allgather(comm.ctx, params.ptr_array, 0, n, 0, shard_grad.data_ptr(),
                                                   master.data_ptr(), m.data_ptr(), v.data_ptr(), flags.data_ptr(),
                                                   hyper.data_ptr(), 0.1, CH_STEP_DONE, 1, ub, stream), "update")
        _native.check(lib.idrak_comm_wait(comm.ctx, CH_STEP_DONE, 0, stream), "wait")

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    rows = []
    for name, fn, hbm_bytes, link_bytes, blocks in (
            ("dp_reduce_scatter_kernel", reduce_scatter, sl * 2 + sl * 4, (world - 1) * sl * 2, a.blocks),
            ("dp_adamw_allgather_kernel", update, sl * 28 + sl * 2, (world - 1) * sl * 2, ub)):
        ms = timed(fn)
        floor_ms = max(hbm_bytes / (hbm * 1e6), link_bytes / (a.nvlink_gbs * 1e6))
        rows.append({"kernel": name, "ranks": world, "bucket_mb": round(n * 2 / 2 ** 20, 1), "blocks": blocks,
                     "ms": round(ms, 4), "hbm_gb_s": round(hbm_bytes / ms / 1e6, 1),
                     "nvlink_gb_s_per_direction": round(link_bytes / ms / 1e6, 1), "roofline_ms": round(floor_ms, 4),
                     "of_roofline": round(floor_ms / ms, 3), "hbm_peak_gbs": hbm, "nvlink_peak_gbs": a.nvlink_gbs,
                     "note": "includes the epoch bump launch and, for the update, the closing step-done wait"})
    _native.check_status("dp_bench")
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    grads.close()
    params.close()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
