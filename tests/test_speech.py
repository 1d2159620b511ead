"""The CTC speech trainer on synthetic "speech": utterances are runs of tones, one pitch per token."""
import math

import torch

from idrak_b200.audio.speech import AcousticModel, SpeechTrainer, edit_distance, token_error_rate

RATE, TOKENS = 8000, 6


def utterance(g: torch.Generator):
    n = int(torch.randint(2, 6, (), generator=g))
    tokens = (torch.randint(0, TOKENS, (n,), generator=g) + 1).tolist()
    parts = []
    for t in tokens:
        length = int(RATE * (0.08 + 0.04 * torch.rand((), generator=g).item()))
        time = torch.arange(length) / RATE
        parts.append(0.5 * torch.sin(2 * math.pi * (300.0 + 350.0 * t) * time))
        parts.append(torch.zeros(int(RATE * 0.02)))
    wave = torch.cat(parts)
    return wave + 0.02 * torch.randn(wave.shape, generator=g), tokens


def test_error_rates():
    assert edit_distance([1, 2, 3], [1, 3]) == 1 and edit_distance([], [4, 5]) == 2 and edit_distance([7], [7]) == 0
    assert token_error_rate([[1, 2], [3]], [[1, 2], [4]]) == 1 / 3
    assert AcousticModel.frames_after(torch.tensor([100, 7, 1])).tolist() == [25, 2, 1]


def test_trainer_learns_the_tone_alphabet():
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1)
    data = [utterance(g) for _ in range(300)]
    held = [utterance(g) for _ in range(40)]
    trainer = SpeechTrainer(AcousticModel(mels=32, classes=TOKENS + 1, width=32, hidden=32), rate=RATE, mels=32, lr=5e-3)
    losses = trainer.fit([w for w, _ in data], [t for _, t in data], steps=220, batch=16)
    assert losses[-1] < 0.5 * losses[0]
    rate = trainer.evaluate([w for w, _ in held], [t for _, t in held])
    assert rate < 0.15, rate
    wave, tokens = held[0]
    assert trainer.transcribe(wave) == trainer.transcribe([wave])[0]
    assert edit_distance(trainer.transcribe(wave, beam=4), tokens) <= 1
