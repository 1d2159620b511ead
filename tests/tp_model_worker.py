"""Worker run under torchrun by the tensor-parallel model tests: trains a small decoder sliced over the ranks for a
few steps and writes losses plus the re-assembled weights of rank 0's view, so the launcher can compare with the
unsliced model. Not collected by pytest.

argv: device ("cpu" | "cuda"), mode ("fused" | "nccl"), family ("llama" | "gpt2"), out path, steps"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_spec(family):
    from idrak_b200.models import DecoderSpec
    if family == "gpt2":
        return DecoderSpec.gpt2(layers=2, dim=256, heads=4, vocab=1000, max_positions=128)
    return DecoderSpec.llama(layers=2, dim=256, heads=4, kv_heads=2, ff_dim=512, vocab=1000, max_positions=128)


def make_data(steps, batch=4, seq=128):
    g = torch.Generator().manual_seed(100)
    return torch.randint(0, 1000, (steps, batch, seq + 1), generator=g)


def main():
    device, mode, family, out_path, steps = sys.argv[1], sys.argv[2], sys.argv[3], sys.argv[4], int(sys.argv[5])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200 import _native
    from idrak_b200.models import build_decoder
    from idrak_b200.parallel.tp import TensorParallel
    from idrak_b200.parallel.tp_layers import TPDecoder, TPOptimizer

    spec = make_spec(family)
    full = build_decoder(spec, seed=7).to(dev, dtype)
    if mode == "fused":
        from idrak_b200.parallel.comm import Communicator
        comm = Communicator(device=dev)
        tp = TensorParallel(comm, max_rows=4 * 128, max_in=1024, max_out=1024)
    else:
        tp = TensorParallel(mode="nccl")
    model = TPDecoder.from_decoder(full, tp)
    del full
    opt = TPOptimizer(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    data = make_data(steps)
    losses = []
    for s in range(steps):
        b = data[s].to(dev)
        opt.zero_grad()
        loss = model.loss(b[:, :-1].contiguous().int(), b[:, 1:].contiguous().int())
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
    if device == "cuda":
        torch.cuda.synchronize()
        _native.check_status("tp_model_worker")
    # a few tensors re-assembled from the shards, to compare with the unsliced run
    def gather_rows(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts, 0)
    embed = gather_rows(model.embed.detach().float())
    down0 = gather_rows(model.blocks[0].down_weight.detach().float().t().contiguous()).t().contiguous()
    norm = model.norm.weight.detach().float()
    if rank == 0:
        torch.save({"losses": losses, "embed": embed.cpu(), "down0": down0.cpu(), "norm": norm.cpu()}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
