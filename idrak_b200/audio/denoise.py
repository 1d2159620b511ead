"""Recurrent noise suppression in the style of RNNoise: a small GRU network looks at coarse band energies of each
frame and predicts a gain per band (and whether the frame holds speech); the gains, interpolated to the FFT bins, scale
the noisy spectrum.

* ``band_matrix``: overlapping triangular bands on an equivalent-rectangular-bandwidth-like scale (dense below 1 kHz,
  wide above), ``[bands, bins]``; its transpose spreads band gains back over the bins;
* ``features``: log band energies, their first and second differences over time for the lowest bands and a
  spectral-variability term - 2 x ``delta_bands`` + ``bands`` + 1 numbers per frame;
* ``Denoiser``: dense -> three GRUs (activity, noise estimate, gains) wired as in RNNoise (each later GRU also sees the
  earlier outputs and the input features) -> sigmoid band gains and an activity probability; every part is causal (one-directional
  GRUs, backward differences), ``forward`` runs whole recordings;
* ``ideal_gains`` / ``denoise_loss``: the training target sqrt(clean band energy / noisy band energy) and RNNoise's loss
  on gains (squared and fourth-power error of the square-rooted gains, activity cross entropy);
* ``DenoiseTrainer``: mixes clean recordings with noise at random signal-to-noise ratios and fits the network.

The GRUs are ``nn/layers.py: Recurrent`` and run on this package's recurrent kernels on CUDA.

Reference: the RNNoise plugin of the audio stack (src/Idrak.Audio, src/Idrak.Plugins).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.layers import Recurrent


def band_matrix(rate: int, n_fft: int, bands: int = 22) -> torch.Tensor:
    """``[bands, n_fft // 2 + 1]`` triangular, overlapping bands whose weights sum to one in every bin."""
    bins = n_fft // 2 + 1
    erb = lambda f: 21.4 * math.log10(1 + 0.00437 * f)
    inv = lambda e: (10 ** (e / 21.4) - 1) / 0.00437
    centres = torch.tensor([inv(erb(0.0) + (erb(rate / 2) - erb(0.0)) * i / (bands - 1)) for i in range(bands)])
    freqs = torch.linspace(0, rate / 2, bins)
    m = torch.zeros(bands, bins)
    for b in range(bands):
        lo = centres[b - 1] if b > 0 else centres[0] - 1.0
        hi = centres[b + 1] if b < bands - 1 else centres[-1] + 1.0
        up = ((freqs - lo) / (centres[b] - lo)).clamp(0, 1)
        down = ((hi - freqs) / (hi - centres[b])).clamp(0, 1)
        m[b] = torch.minimum(up, down)
    m[0, freqs <= centres[0]] = 1.0
    m[-1, freqs >= centres[-1]] = 1.0
    return m / m.sum(0, keepdim=True).clamp_min(1e-8)


def band_energies(spec: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """``spec`` complex ``[B, bins, T]`` -> band energies ``[B, T, bands]``."""
    power = spec.real ** 2 + spec.imag ** 2
    return (matrix.to(power) @ power).transpose(1, 2)


def features(energies: torch.Tensor, delta_bands: int = 6) -> torch.Tensor:
    """``[B, T, bands]`` energies -> ``[B, T, bands + 2 delta_bands + 1]`` features (causal differences)."""
    log_e = torch.log10(energies + 1e-3)
    low = log_e[..., :delta_bands]
    prev = F.pad(low, (0, 0, 1, 0))[:, :-1]
    prev2 = F.pad(low, (0, 0, 2, 0))[:, :-2]
    d1, d2 = low - prev, low - 2 * prev + prev2
    # how much the band shape moves against the recent past (eight frames): small for stationary noise
    hist = torch.stack([F.pad(log_e, (0, 0, k, 0))[:, :log_e.shape[1]] for k in range(1, 9)], 0)
    variability = ((log_e[None] - hist) ** 2).sum(-1).min(0).values.unsqueeze(-1) / log_e.shape[-1]
    return torch.cat([log_e, d1, d2, variability], -1)


class Denoiser(nn.Module):
    def __init__(self, rate: int = 48000, n_fft: int = 960, bands: int = 22, delta_bands: int = 6,
                 sizes: Tuple[int, int, int, int] = (24, 24, 48, 96)):
        super().__init__()
        self.rate, self.n_fft, self.hop, self.bands, self.delta_bands = rate, n_fft, n_fft // 2, bands, delta_bands
        n_in = bands + 2 * delta_bands + 1
        dense, vad, noise, gain = sizes
        self.register_buffer("matrix", band_matrix(rate, n_fft, bands), persistent=False)
        self.input_dense = nn.Linear(n_in, dense)
        self.vad_gru = Recurrent("gru", dense, vad, sequences=True)
        self.vad_out = nn.Linear(vad, 1)
        self.noise_gru = Recurrent("gru", dense + vad + n_in, noise, sequences=True)
        self.gain_gru = Recurrent("gru", vad + noise + n_in, gain, sequences=True)
        self.gain_out = nn.Linear(gain, bands)

    # -------------------------------------------------------------------------------------------------- the network
    def gains(self, feats: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[B, T, features]`` -> (band gains ``[B, T, bands]`` in (0, 1), speech probability ``[B, T]``)."""
        x = torch.tanh(self.input_dense(feats))
        v = self.vad_gru(x)
        n = self.noise_gru(torch.cat([x, v, feats], -1))
        g = self.gain_gru(torch.cat([v, n, feats], -1))
        return torch.sigmoid(self.gain_out(g)), torch.sigmoid(self.vad_out(v))[..., 0]

    def analyse(self, wave: torch.Tensor) -> torch.Tensor:
        window = torch.hann_window(self.n_fft, device=wave.device).sqrt()          # square-root Hann at 50 % overlap:
        return torch.stft(wave.float(), self.n_fft, self.hop, self.n_fft, window,   # analysis x synthesis sums to one
                          center=True, pad_mode="reflect", return_complex=True)

    def synthesise(self, spec: torch.Tensor, length: int) -> torch.Tensor:
        window = torch.hann_window(self.n_fft, device=spec.device).sqrt()
        return torch.istft(spec, self.n_fft, self.hop, self.n_fft, window, center=True, length=length)

    def forward(self, wave: torch.Tensor, floor: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
        """Noisy recordings ``[B, samples]`` -> (denoised ``[B, samples]``, speech probability per frame ``[B, T]``)."""
        spec = self.analyse(wave)
        g, vad = self.gains(features(band_energies(spec, self.matrix), self.delta_bands))
        bin_gain = (g.clamp_min(floor) @ self.matrix.to(g)).transpose(1, 2)         # [B, bins, T]
        return self.synthesise(spec * bin_gain, wave.shape[-1]), vad


def ideal_gains(clean_energy: torch.Tensor, noisy_energy: torch.Tensor) -> torch.Tensor:
    return torch.sqrt(clean_energy / noisy_energy.clamp_min(1e-9)).clamp(0, 1)


def denoise_loss(gains: torch.Tensor, vad: torch.Tensor, target_gains: torch.Tensor, target_vad: torch.Tensor) -> torch.Tensor:
    """RNNoise's objective: errors of the square-rooted gains, squared and (ten times) to the fourth power, plus half the
    activity cross entropy."""
    diff = torch.sqrt(gains.clamp_min(1e-9)) - torch.sqrt(target_gains.clamp_min(1e-9))
    return (diff ** 2).mean() + 10 * (diff ** 4).mean() + 0.5 * F.binary_cross_entropy(vad, target_vad)


class DenoiseTrainer:
    def __init__(self, model: Denoiser, lr: float = 1e-3, snr_db: Tuple[float, float] = (-5.0, 20.0), seed: int = 0):
        self.model = model
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr)
        self.snr_db = snr_db
        self.generator = torch.Generator().manual_seed(seed)
        self.steps = 0

    def mix(self, clean: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
        """Clean + noise scaled to a signal-to-noise ratio drawn per recording."""
        lo, hi = self.snr_db
        snr = lo + (hi - lo) * torch.rand(clean.shape[0], generator=self.generator).to(clean.device)
        scale = torch.sqrt(clean.pow(2).mean(-1) / (noise.pow(2).mean(-1).clamp_min(1e-9) * 10 ** (snr / 10)))
        return clean + noise * scale[:, None]

    def step(self, clean: torch.Tensor, noise: torch.Tensor) -> Dict[str, float]:
        m = self.model
        noisy = self.mix(clean, noise)
        e_clean = band_energies(m.analyse(clean), m.matrix)
        e_noisy = band_energies(m.analyse(noisy), m.matrix)
        target = ideal_gains(e_clean, e_noisy)
        frame_energy = e_clean.sum(-1)
        active = (frame_energy > 0.01 * frame_energy.amax(-1, keepdim=True)).float()
        g, vad = m.gains(features(e_noisy, m.delta_bands))
        loss = denoise_loss(g, vad, target, active)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        self.steps += 1
        return {"loss": float(loss.detach())}


def snr_db(clean: torch.Tensor, estimate: torch.Tensor) -> torch.Tensor:
    """Signal-to-noise ratio of ``estimate`` against ``clean`` per recording, in decibels."""
    err = (estimate - clean).pow(2).sum(-1).clamp_min(1e-12)
    return 10 * torch.log10(clean.pow(2).sum(-1).clamp_min(1e-12) / err)
