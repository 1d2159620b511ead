"""FineTuner on the device: the recorded (CUDA graph) step against the eager step, and the packed bases."""
import pytest
import torch

from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.text import ByteTokenizer
from idrak_b200.text.finetuning import FineTuner, FineTuningOptions

pytestmark = pytest.mark.gpu


def _model(seed=1):
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=128, heads=2, kv_heads=1, ff_dim=256, vocab=tok.vocab_size, max_positions=512)
    model = build_decoder(spec, seed=seed).to("cuda", torch.bfloat16)
    return model, tok


def _examples(n=24):
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta"]
    return [{"prompt": f"say {words[i % 6]} {i % 5} times: ", "response": " ".join([words[i % 6]] * (1 + i % 5))}
            for i in range(n)]


def _run(capture: bool, base="bf16"):
    model, tok = _model()
    o = FineTuningOptions(rank=16, learning_rate=2e-3, batch_tokens=256, max_length=128, max_steps=12, base=base,
                          capture_graph=capture, activation_ladder=False, seed=3)
    tuner = FineTuner(model, tok, o)
    res = tuner.fit(_examples())
    return res, [p.detach().float().clone() for p in tuner.params]


def test_recorded_step_follows_the_eager_step():
    eager, p0 = _run(False)
    graphed, p1 = _run(True)
    assert eager.graph_replays == 0 and graphed.graph_replays >= 9          # two eager warm-up steps, then replays
    assert graphed.steps == eager.steps == 12 and graphed.skipped_steps == 0
    # the padded tail is a sequence of its own with no trained token: the losses agree to bf16 noise
    for a, b in zip(eager.losses, graphed.losses):
        assert abs(a - b) < 0.05 * max(1.0, abs(a)), (eager.losses, graphed.losses)
    assert graphed.losses[-1] < graphed.losses[0]
    moved = max((a - b).abs().max().item() for a, b in zip(p0, p1))
    assert moved < 0.05, moved


@pytest.mark.parametrize("base", ["int8", "int4"])
def test_packed_bases_train_with_fused_adapters(base):
    res, _ = _run(False, base)
    assert res.steps == 12 and all(map(lambda v: v == v and v < 20, res.losses))
    assert res.losses[-1] < res.losses[0]
