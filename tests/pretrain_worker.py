"""Worker run under torchrun by the pre-training tests (gloo CPU ranks). Not collected by pytest.
argv: token file, out dir, steps, resume folder or '-'"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    tokens, out_dir, steps, resume = sys.argv[1], sys.argv[2], int(sys.argv[3]), sys.argv[4]
    dist.init_process_group("gloo")
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.text.pretraining import PretrainOptions, PretrainStage, Pretrainer
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=300, max_positions=64)
    model = build_decoder(spec, seed=3).float()
    o = PretrainOptions(stages=[PretrainStage("a", [tokens], steps=steps, seq_len=32)], global_batch=8, micro_batch=2,
                        learning_rate=3e-3, warmup_steps=2, out_dir=out_dir, resume_from=None if resume == "-" else resume,
                        seed=11)
    res = Pretrainer.train(model, o)
    if dist.get_rank() == 0:
        with open(os.path.join(out_dir, "losses.json"), "w") as f:
            json.dump(res.losses, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
