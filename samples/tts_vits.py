"""Text to speech with VITS. With ``--model <folder>`` (a Hugging Face VITS folder with ``config.json`` and
``model.safetensors``) the text is spoken with the checkpoint's
voice. Without one, a small model of the same architecture is trained for a few steps on a synthetic corpus (each
"letter" is a tone of its own pitch, a "word" is the tones in sequence) and then asked to say a new word, so that the
whole path - alignment search, posterior / prior / flow, generator, duration model, waveform file - runs offline.

    python samples/tts_vits.py [--model <folder>] [--text "hello"] [--out speech.wav] [--steps 60] [--adversarial]

Reference: samples/OpenVoice and the VITS plugin's text-to-speech entry.
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.audio import write_wav  # noqa: E402
from idrak_b200.audio.vits import Discriminators, Vits, VitsSpec, VitsTrainer  # noqa: E402

ALPHABET = "_abcdefgh"                                    # id 0 pads
RATE = 8000


def tone_word(word: str, hop: int, frames_per_letter: int = 6) -> torch.Tensor:
    """Each letter: ``frames_per_letter`` frames of a sine at 200 Hz + 90 Hz per letter index."""
    n = frames_per_letter * hop
    t = torch.arange(n) / RATE
    return torch.cat([0.5 * torch.sin(2 * math.pi * (200 + 90 * ALPHABET.index(ch)) * t) for ch in word])


def corpus(hop: int, words=("abc", "cab", "hedge", "bead", "fade", "gabe", "chafe", "badge")):
    ids = [torch.tensor([ALPHABET.index(c) for c in w]) for w in words]
    waves = [tone_word(w, hop) for w in words]
    T, S = max(len(i) for i in ids), max(len(w) for w in waves)
    pad = lambda x, n: torch.cat([x, x.new_zeros(n - len(x))])
    return (torch.stack([pad(i, T) for i in ids]), torch.tensor([len(i) for i in ids]),
            torch.stack([pad(w, S) for w in waves]), torch.tensor([len(w) for w in waves]))


def load(folder: str) -> Vits:
    from idrak_b200.formats.safetensors import load_file
    with open(os.path.join(folder, "config.json")) as f:
        model = Vits(VitsSpec.from_hf(json.load(f)))
    model.load_hf_state(load_file(os.path.join(folder, "model.safetensors")))
    return model


def main(model_folder=None, text="badge", out=None, steps=60, adversarial=False, device="cpu", quiet=False) -> dict:
    say = (lambda *a: None) if quiet else print
    if model_folder:
        model = load(model_folder).to(device).eval()
        with open(os.path.join(model_folder, "vocab.json")) as f:
            vocab = json.load(f)
        ids = torch.tensor([[vocab[c] for c in text.lower() if c in vocab]], device=device)
        history = []
    else:
        torch.manual_seed(0)
        spec = VitsSpec(vocab_size=len(ALPHABET), hidden=32, layers=2, heads=2, window=2, ffn=64, flow_size=16,
                        spectrogram_bins=65, duration_filter=32, prior_flows=2, prior_wavenet_layers=2,
                        posterior_wavenet_layers=3, wavenet_kernel=3, upsample_rates=(4, 4, 2), upsample_kernels=(8, 8, 4),
                        upsample_channels=64, resblock_kernels=(3, 5), resblock_dilations=((1, 3), (1, 2)),
                        sampling_rate=RATE, noise_scale=0.3)
        model = Vits(spec).to(device)
        disc = Discriminators(periods=(2, 3, 5), period_channels=(8, 16, 32), scale_width=4).to(device) if adversarial else None
        trainer = VitsTrainer(model, disc, lr=2e-3, segment=12)
        batch = [t.to(device) for t in corpus(spec.hop)]
        history = []
        for step in range(steps):
            report = trainer.step(*batch)
            history.append(report)
            if step % 10 == 0 or step == steps - 1:
                say(f"step {step:3d}  spectral {report['spectral']:.3f}  kl {report['kl']:.3f}  duration {report['duration']:.3f}"
                    + (f"  disc {report['discriminator']:.3f}" if adversarial else ""))
        model.eval()
        ids = torch.tensor([[ALPHABET.index(c) for c in text if c in ALPHABET[1:]]], device=device)
    wave, samples = model.synthesize(ids, generator=torch.Generator(device=device).manual_seed(1))
    wave = wave[0, :int(samples[0])].float().cpu()
    rate = model.spec.sampling_rate
    say(f"{ids.shape[1]} tokens -> {len(wave)} samples ({len(wave) / rate:.2f} s at {rate} Hz), peak {wave.abs().max():.2f}")
    if out:
        write_wav(out, wave.clamp(-1, 1), rate)
        say("wrote", out)
    return {"samples": len(wave), "rate": rate, "history": history, "wave": wave}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--text", default="badge")
    ap.add_argument("--out")
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--adversarial", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    main(a.model, a.text, a.out, a.steps, a.adversarial, a.device)
