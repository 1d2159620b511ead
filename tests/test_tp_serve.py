"""Tensor-parallel serving: sharding on the CPU, and the 2-rank engine against the unsplit model on GPUs."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def test_sharded_blocks_sum_to_the_whole_model_on_cpu():
    from idrak_b200.models import DecoderSpec, build_decoder
    from idrak_b200.parallel.tp_serve import check_shardable, local_spec, shard_decoder, vocab_slice
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=250, max_positions=64)
    full = build_decoder(spec, seed=1).eval()
    parts = [shard_decoder(full, r, 2) for r in range(2)]
    ls = local_spec(spec, 2)
    assert (ls.heads, ls.kv_heads, ls.ff_dim, ls.dim, ls.head_dim) == (2, 1, 64, 64, spec.head_dim)
    x = torch.randn(1, 5, 64)
    # feed-forward: column slices of gate / up and row slices of down add up to the whole layer
    whole = full.blocks[0].mlp(x)
    assert torch.allclose(sum(p.blocks[0].mlp(x) for p in parts), whole, atol=1e-5)
    # attention: each rank's heads, summed after the output projection
    h = full.blocks[0].attn_norm(x)
    whole = full.blocks[0].attn(h)
    assert torch.allclose(sum(p.blocks[0].attn(h) for p in parts), whole, atol=1e-5)
    # the head: vocabulary rows side by side
    hid = full.norm(x)
    logits = torch.cat([torch.nn.functional.linear(hid, p.tp_head) for p in parts], -1)[..., :250]
    assert torch.allclose(logits, full.forward_from_hidden(hid), atol=1e-5)
    assert vocab_slice(spec, 1, 2) == (spec.padded_vocabulary // 2, spec.padded_vocabulary)
    with pytest.raises(ValueError, match="do not divide"):
        check_shardable(spec, 3)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_rank_engine_matches_the_unsplit_model(tmp_path):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = tmp_path / "tp_serve.pt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29647", os.path.join(HERE, "tp_serve_worker.py"), str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    ok = torch.load(out)
    bad = [k for k, v in ok.items() if v is False]
    assert not bad, (bad, ok)
