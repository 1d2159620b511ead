"""Rank process (gloo, CPU) of the fine-tuner's flat data-parallel test: each rank trains on its share of the examples
with one gradient all-reduce per step; rank 0 writes whether the ranks started and ended with equal adapters. Not
collected by pytest."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from idrak_b200.adapters.lora import adapter_parameters
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.text import ByteTokenizer
    from idrak_b200.text.finetuning import FineTuner, FineTuningOptions
    torch.manual_seed(100 + rank)                  # whatever a rank drew before must not reach the adapters
    torch.rand(rank + 1)
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=64, heads=2, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=256)
    model = build_decoder(spec, seed=1).float()
    examples = [{"prompt": f"say {w} twice: ", "response": f"{w} {w}"} for w in
                ("alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta")]
    opts = FineTuningOptions(rank=8, alpha=16.0, learning_rate=2e-3, max_steps=4, batch_tokens=128, seed=3,
                             data_parallel="flat", activation_ladder=False)
    tuner = FineTuner(model, tok, opts)

    def same():
        flat = torch.cat([p.detach().float().reshape(-1) for p in adapter_parameters(model)])
        parts = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(parts, flat)
        return all(torch.equal(parts[0], p) for p in parts)

    start = same()
    res = tuner.fit(examples[rank::world])
    end = same()
    if rank == 0:
        torch.save({"start": start, "end": end, "losses": res.losses}, out)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
