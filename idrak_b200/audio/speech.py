"""Speech recognition with connectionist temporal classification: a log-mel front end, a small convolutional-recurrent
acoustic model, a trainer (``SpeechTrainer``) that pads batches, tracks the frame counts the convolutions leave, clips
gradients and reports the token error rate, and greedy / beam decoding of the result.

    model = AcousticModel(mels=40, classes=len(alphabet) + 1)
    trainer = SpeechTrainer(model, rate=8000)
    trainer.fit(waveforms, transcripts, steps=300)          # transcripts: lists of token ids >= 1 (0 is the blank)
    ids = trainer.transcribe(waveform)

On a GPU the convolutions, the recurrent cells and the CTC loss run on the package's kernels.

Reference: the CTC speech trainers (src/Idrak.Audio/Speech: acoustic model training loop, error rates, decoding).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn

from . import MelSpec, ctc_beam, ctc_greedy, log_mel
from ..nn import layers as L
from ..nn.losses import ctc


class AcousticModel(nn.Module):
    """Two strided 1-D convolutions over the mel bands (time reduced by four), a bidirectional GRU, class scores."""

    def __init__(self, mels: int = 40, classes: int = 32, width: int = 64, hidden: int = 64):
        super().__init__()
        self.conv = nn.Sequential(L.Conv1d(mels, width, 5, stride=2, padding=2), nn.ReLU(),
                                  L.Conv1d(width, width, 5, stride=2, padding=2), nn.ReLU())
        self.rnn = L.Recurrent("gru", width, hidden, sequences=True, bidirectional=True)
        self.head = L.Linear(2 * hidden, classes)

    @staticmethod
    def frames_after(frames: torch.Tensor) -> torch.Tensor:
        """How many output steps ``frames`` input frames leave (two convolutions of stride 2, kernel 5, padding 2)."""
        for _ in range(2):
            frames = (frames + 2 * 2 - 5) // 2 + 1
        return frames

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """``[N, mels, frames]`` -> scores ``[N, steps, classes]``."""
        return self.head(self.rnn(self.conv(mel).transpose(1, 2)))


def edit_distance(a: Sequence[int], b: Sequence[int]) -> int:
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


def token_error_rate(predicted: Sequence[Sequence[int]], truth: Sequence[Sequence[int]]) -> float:
    """Edit distance summed over the utterances, over the number of reference tokens."""
    errors = sum(edit_distance(p, t) for p, t in zip(predicted, truth))
    return errors / max(1, sum(len(t) for t in truth))


class SpeechTrainer:
    def __init__(self, model: AcousticModel, rate: int = 16000, mels: int = 40, lr: float = 3e-3, clip: float = 5.0,
                 device: Optional[str] = None, seed: int = 0):
        self.model, self.rate, self.clip, self.seed = model, rate, clip, seed
        self.device = torch.device(device) if device else next(model.parameters()).device
        self.model.to(self.device)
        n_fft = 256 if rate <= 8000 else 400
        self.spec = MelSpec(rate=rate, n_fft=n_fft, hop=n_fft // 4, n_mels=mels, f_min=0.0, f_max=rate / 2, log="ln")
        self.optimizer = torch.optim.Adam(model.parameters(), lr=lr)
        self.losses: List[float] = []

    def features(self, waves: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """Padded log-mel batch ``[N, mels, frames]`` (per-utterance mean removed) and the frame count of each."""
        mels = [log_mel(w.float().reshape(-1), self.spec) for w in waves]
        mels = [m - m.mean() for m in mels]
        frames = torch.tensor([m.shape[-1] for m in mels])
        batch = torch.zeros(len(mels), mels[0].shape[0], int(frames.max()))
        for i, m in enumerate(mels):
            batch[i, :, : m.shape[-1]] = m
        return batch, frames

    def step(self, waves: Sequence[torch.Tensor], transcripts: Sequence[Sequence[int]]) -> float:
        mel, frames = self.features(waves)
        longest = max(len(t) for t in transcripts)
        targets = torch.zeros(len(transcripts), max(longest, 1), dtype=torch.long)
        for i, t in enumerate(transcripts):
            targets[i, : len(t)] = torch.tensor(list(t), dtype=torch.long)
        lengths = torch.tensor([len(t) for t in transcripts])
        self.model.train()
        scores = self.model(mel.to(self.device))
        log_probs = torch.log_softmax(scores.float(), -1).transpose(0, 1)            # [T, N, C]
        steps = AcousticModel.frames_after(frames).clamp(max=log_probs.shape[0])
        loss = ctc(log_probs, targets.to(self.device), steps.to(self.device), lengths.to(self.device))
        self.optimizer.zero_grad()
        loss.backward()
        nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)
        self.optimizer.step()
        self.losses.append(float(loss.detach()))
        return self.losses[-1]

    def fit(self, waves: Sequence[torch.Tensor], transcripts: Sequence[Sequence[int]], steps: int = 300, batch: int = 16,
            progress=None) -> List[float]:
        g = torch.Generator().manual_seed(self.seed)
        for k in range(steps):
            idx = torch.randint(0, len(waves), (batch,), generator=g).tolist()
            value = self.step([waves[i] for i in idx], [transcripts[i] for i in idx])
            if progress:
                progress(k + 1, value)
        return self.losses

    @torch.no_grad()
    def transcribe(self, waves, beam: int = 0) -> List[List[int]]:
        single = torch.is_tensor(waves)
        batch = [waves] if single else list(waves)
        mel, frames = self.features(batch)
        self.model.eval()
        log_probs = torch.log_softmax(self.model(mel.to(self.device)).float(), -1).cpu()
        steps = AcousticModel.frames_after(frames).clamp(max=log_probs.shape[1]).tolist()
        if beam > 1:
            out = [ctc_beam(log_probs[i, : steps[i]], beam)[0] for i in range(len(batch))]
        else:
            out = ctc_greedy(log_probs, 0, steps)
        return out[0] if single else out

    def evaluate(self, waves, transcripts) -> float:
        return token_error_rate(self.transcribe(list(waves)), transcripts)
