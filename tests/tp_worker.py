"""Worker run under torchrun by the tensor-parallel tests: runs the fused all-gather->GEMM and GEMM->reduce-scatter
kernels on every rank against a plain fp32 statement of the same math and writes the largest errors. Not collected
by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, rounds = sys.argv[1], int(sys.argv[2])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200 import _native
    from idrak_b200.parallel.comm import Communicator
    from idrak_b200.parallel.tp import TensorParallel

    comm = Communicator(device=dev)
    M, K, N = 256 * world, 320, 384               # rows_per_rank = 256 (two chunks); N spans two column tiles
    tp = TensorParallel(comm, max_rows=M, max_in=max(K, N), max_out=max(K, N))
    g = torch.Generator().manual_seed(5)          # same numbers on every rank: each takes its slice
    errs = {"ag": 0.0, "ag_gelu": 0.0, "ag_mn": 0.0, "rs": 0.0, "rs_mn": 0.0}
    for it in range(rounds):
        X = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
        W = (torch.randn(world * N, K, generator=g) * 0.1).to(torch.bfloat16)      # column-parallel: N per rank
        b = torch.randn(world * N, generator=g).to(torch.bfloat16)
        rows = M // world
        x_local = X[rank * rows:(rank + 1) * rows].to(dev)
        w_local = W[rank * N:(rank + 1) * N].to(dev)
        b_local = b[rank * N:(rank + 1) * N].to(dev)
        ref = X.float() @ W[rank * N:(rank + 1) * N].float().t() + b[rank * N:(rank + 1) * N].float()
        y = tp.ag_gemm(x_local, w_local, bias=b_local)
        errs["ag"] = max(errs["ag"], (y.float().cpu() - ref).abs().max().item())
        y2, pre = tp.ag_gemm(x_local, w_local, bias=b_local, act="gelu")
        errs["ag_gelu"] = max(errs["ag_gelu"], (pre.float().cpu() - ref).abs().max().item(),
                              (y2.float().cpu() - torch.nn.functional.gelu(ref, approximate="tanh")).abs().max().item())
        w_kn = w_local.t().contiguous()                                          # stored [K, N]
        y3 = tp.ag_gemm(x_local, w_kn, w_mn=True)
        errs["ag_mn"] = max(errs["ag_mn"], (y3.float().cpu() - (ref - b[rank * N:(rank + 1) * N].float())).abs().max().item())
        # row-parallel: every rank holds K columns of a [M, world * K] input and of the [N, world * K] weight
        Xr = (torch.randn(M, world * K, generator=g) * 0.5).to(torch.bfloat16)
        Wr = (torch.randn(N, world * K, generator=g) * 0.1).to(torch.bfloat16)
        res = torch.randn(M, N, generator=g).to(torch.bfloat16)
        br = torch.randn(N, generator=g).to(torch.bfloat16)
        xs = Xr[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        ws = Wr[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        # the kernel sums bf16-rounded partial products in rank order
        parts = [(Xr[:, r * K:(r + 1) * K].float() @ Wr[:, r * K:(r + 1) * K].float().t()).to(torch.bfloat16).float()
                 for r in range(world)]
        full = sum(parts) + br.float() + res.float()
        mine = slice(rank * rows, (rank + 1) * rows)
        o = tp.gemm_rs(xs, ws, bias=br.to(dev), residual=res[mine].to(dev))
        errs["rs"] = max(errs["rs"], (o.float().cpu() - full[mine]).abs().max().item())
        o2 = tp.gemm_rs(xs, ws.t().contiguous(), w_mn=True)
        errs["rs_mn"] = max(errs["rs_mn"], (o2.float().cpu() - sum(parts)[mine]).abs().max().item())
    torch.cuda.synchronize()
    _native.check_status("tp_worker")
    seq = int(tp.state[0].item())
    gathered = [None] * world
    dist.all_gather_object(gathered, errs)
    if rank == 0:
        worst = {k: max(e[k] for e in gathered) for k in errs}
        torch.save({"errors": worst, "seq": seq, "world": world}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
