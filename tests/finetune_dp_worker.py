"""Rank process of the fine-tuner's data-parallel test: a short LoRA run over this rank's share of the examples with
the gradient path given in argv (fused | nccl | flat). Writes the final adapter weights, the losses and how many
kernels of the native library ran. Not collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode, out = sys.argv[1], sys.argv[2]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200 import _native
    from idrak_b200.adapters.lora import adapter_parameters
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.text import ByteTokenizer
    from idrak_b200.text.finetuning import FineTuner, FineTuningOptions
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=128, heads=2, kv_heads=2, ff_dim=256, vocab=tok.vocab_size, max_positions=256)
    spec.head_dim = 64
    model = build_decoder(spec, seed=1).to(dev, torch.bfloat16)
    examples = [{"prompt": f"say {w} twice: ", "response": f"{w} {w}"} for w in
                ("alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta")]
    mine = examples[rank::world]
    opts = FineTuningOptions(rank=8, alpha=16.0, learning_rate=2e-3, max_steps=6, batch_tokens=128, seed=3,
                             data_parallel=mode, activation_ladder=False)
    tuner = FineTuner(model, tok, opts)
    before = _native.lib().idrak_launch_count()
    res = tuner.fit(mine)
    torch.cuda.synchronize()
    _native.check_status("finetune worker")
    launches = _native.lib().idrak_launch_count() - before
    flat = torch.cat([p.detach().float().reshape(-1) for p in adapter_parameters(model)])
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    if rank == 0:
        torch.save({"weights": flat.cpu(), "losses": res.losses, "launches": launches, "sync": type(tuner.sync).__name__,
                    "same": all(torch.equal(parts[0], p) for p in parts)}, out)
    if tuner.sync is not None:
        tuner.sync.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
