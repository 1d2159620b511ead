"""Times the fused tensor-parallel kernels against NCCL collective + GEMM on the projections of a decoder layer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29700 \
        -m idrak_b200.diag.tp_bench --tokens 8192 --dim 4096 --heads 32 --kv-heads 8 --ff 14336

For each projection (QKV, attention output, MLP up, MLP down) rank 0 prints one JSON line: milliseconds of the
fused kernel and of the unfused pair (max over ranks, CUDA events, warm-up first), the roofline time
``max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s)`` and the fraction of it each reaches.

Reference: the cluster bandwidth probe of the reference (src/Idrak.Network/Diagnostics) reports link and collective
times the same way; it has no fused compute + collective kernels to compare.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

GEMM_PEAK_TFLOPS = 1396.6        # sustained cuBLAS bf16 on this machine class
LINK_GBS = 770.0                 # measured peer copy bandwidth per direction


def _time(fn, warmup, iters, group):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
    return float(ms.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--ff", type=int, default=14336)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--push-ctas", type=int, default=16)
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from .. import _native, ops
    from ..parallel.comm import Communicator
    from ..parallel.tp import TensorParallel

    M, dim = a.tokens, a.dim
    qkv_n = (a.heads + 2 * a.kv_heads) * a.head_dim // world
    o_k = a.heads * a.head_dim // world
    up_n, down_k = 2 * a.ff // world, a.ff // world
    comm = Communicator(device=dev)
    tp = TensorParallel(comm, max_rows=M, max_in=dim, max_out=dim, push_ctas=a.push_ctas)
    base = TensorParallel(mode="nccl")
    rows = M // world
    bf = dict(device=dev, dtype=torch.bfloat16)
    x_local = torch.randn(rows, dim, **bf)
    cases = [
        ("qkv  all-gather->GEMM", "ag", x_local, torch.randn(qkv_n, dim, **bf) * 0.02),
        ("out  GEMM->reduce-scatter", "rs", torch.randn(M, o_k, **bf), torch.randn(dim, o_k, **bf) * 0.02),
        ("up   all-gather->GEMM", "ag", x_local, torch.randn(up_n, dim, **bf) * 0.02),
        ("down GEMM->reduce-scatter", "rs", torch.randn(M, down_k, **bf), torch.randn(dim, down_k, **bf) * 0.02),
    ]
    for name, kind, x, w in cases:
        if kind == "ag":
            fused = lambda: tp.ag_gemm(x, w)
            unfused = lambda: ops.gemm(base.all_gather_rows(x), w)
            N, K = w.shape[0], dim
            flops = 2.0 * M * N * K
            link = (world - 1) / world * M * K * 2           # bytes every rank must receive
        else:
            fused = lambda: tp.gemm_rs(x, w)
            unfused = lambda: base.reduce_scatter_rows(ops.gemm(x, w))
            N, K = dim, x.shape[1]
            flops = 2.0 * M * N * K
            link = (world - 1) / world * M * N * 2           # bytes every rank must send
        t_f = _time(fused, a.warmup, a.iters, None)
        t_u = _time(unfused, a.warmup, a.iters, None)
        roof = max(flops / (GEMM_PEAK_TFLOPS * 1e12), link / (LINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"op": name, "world": world, "multicast": tp.gather_mc is not None, "M": M, "N": N, "K": K, "fused_ms": round(t_f, 4),
                              "nccl_plus_gemm_ms": round(t_u, 4), "speedup": round(t_u / t_f, 3),
                              "roofline_ms": round(roof, 4), "fused_frac_of_roofline": round(roof / t_f, 3),
                              "bound": "compute" if flops / (GEMM_PEAK_TFLOPS * 1e12) > link / (LINK_GBS * 1e9) else "link"}),
                  flush=True)
    torch.cuda.synchronize()
    _native.check_status("tp_bench")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
