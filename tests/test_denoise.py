"""Recurrent noise suppression (``audio/denoise.py``)."""
import math

import torch

from idrak_b200.audio import denoise as D


def test_bands_partition_the_spectrum_and_resynthesis_is_exact():
    m = D.band_matrix(16000, 256, 18)
    assert m.shape == (18, 129)
    torch.testing.assert_close(m.sum(0), torch.ones(129), atol=1e-6, rtol=0)
    peaks = m.argmax(1)
    assert bool((peaks[1:] >= peaks[:-1]).all()) and peaks[1] - peaks[0] < peaks[-1] - peaks[-2]   # wider bands above
    model = D.Denoiser(16000, 256, 18)
    wave = torch.randn(2, 4000)
    back = model.synthesise(model.analyse(wave), 4000)
    torch.testing.assert_close(back, wave, atol=1e-4, rtol=1e-4)
    feats = D.features(D.band_energies(model.analyse(wave), model.matrix), 6)
    assert feats.shape == (2, 4000 // 128 + 1, 18 + 12 + 1)
    # causal: changing the end of the recording leaves the early features alone
    other = wave.clone()
    other[:, 3000:] = 0
    feats2 = D.features(D.band_energies(model.analyse(other), model.matrix), 6)
    torch.testing.assert_close(feats2[:, :20], feats[:, :20])


def test_training_raises_the_signal_to_noise_ratio():
    torch.manual_seed(0)
    rate, n = 16000, 8000
    t = torch.arange(n) / rate
    def voice(f0, on):                                                   # harmonic bursts with silences between
        tone = sum(torch.sin(2 * math.pi * f0 * k * t) / k for k in range(1, 5))
        gate = (torch.sin(2 * math.pi * on * t) > -0.2).float()
        return 0.3 * tone * gate
    clean = torch.stack([voice(140, 3), voice(200, 2), voice(260, 4), voice(180, 5)])
    model = D.Denoiser(rate, 256, 18, sizes=(16, 16, 24, 32))
    trainer = D.DenoiseTrainer(model, lr=5e-3, snr_db=(0.0, 10.0))
    losses = [trainer.step(clean, torch.randn(4, n))["loss"] for _ in range(60)]
    assert losses[-1] < 0.6 * losses[0]
    model.eval()
    noise = torch.randn(4, n, generator=torch.Generator().manual_seed(5))
    noisy = clean + noise * (clean.pow(2).mean(-1) / noise.pow(2).mean(-1) / 10 ** 0.5).sqrt()[:, None]   # 5 dB
    with torch.no_grad():
        cleaned, vad = model(noisy)
    before, after = D.snr_db(clean, noisy), D.snr_db(clean, cleaned)
    assert cleaned.shape == noisy.shape and bool((after > before + 2.0).all()), (before, after)
    # the activity output separates bursts from gaps
    energy = D.band_energies(model.analyse(clean), model.matrix).sum(-1)
    loud = energy > 0.01 * energy.amax(-1, keepdim=True)
    assert vad[loud].mean() > vad[~loud].mean() + 0.2
