"""Audio front end: WAV files, polyphase resampling, STFT, mel filter banks and log-mel features (the Whisper front
end among them), and greedy / prefix-beam CTC decoding. Tensor math runs wherever its input lives (CPU or CUDA).

    samples, rate = read_wav("clip.wav")                   # float32 [channels, n] in -1..1
    mono16k = resample(samples.mean(0), rate, 16000)
    features = log_mel(mono16k, MelSpec.whisper())         # [80, frames]

Reference: src/Idrak.Audio (codecs, Resampler, Stft / MelFilterBank / LogMel features, CTC decoding in the speech
trainers; Whisper front end in src/Idrak.Audio.Plugins). FLAC / MP3 decoding, capture / playback and the TTS stacks
are not built here.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------------------------------
# WAV
# ---------------------------------------------------------------------------------------------------------------------
class AudioFormatError(ValueError):
    pass


def decode_wav(data: bytes) -> Tuple[torch.Tensor, int]:
    """PCM 8 / 16 / 24 / 32-bit integer and 32 / 64-bit float WAV -> (float32 ``[channels, samples]`` in -1..1, rate)."""
    if data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise AudioFormatError("not a RIFF / WAVE file")
    at, fmt, pcm = 12, None, None
    while at + 8 <= len(data):
        tag, size = data[at: at + 4], struct.unpack("<I", data[at + 4: at + 8])[0]
        body = data[at + 8: at + 8 + size]
        if tag == b"fmt ":
            fmt = struct.unpack("<HHIIHH", body[:16])
            if fmt[0] == 0xFFFE and len(body) >= 26:            # extensible: the real format is in the sub-format GUID
                fmt = (struct.unpack("<H", body[24:26])[0],) + fmt[1:]
        elif tag == b"data":
            pcm = body
        at += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise AudioFormatError("WAV without 'fmt ' or 'data'")
    kind, channels, rate, _, _, bits = fmt
    if kind == 1:
        if bits == 8:
            x = (np.frombuffer(pcm, np.uint8).astype(np.float32) - 128.0) / 128.0
        elif bits == 16:
            x = np.frombuffer(pcm, "<i2").astype(np.float32) / 32768.0
        elif bits == 24:
            b = np.frombuffer(pcm[: len(pcm) // 3 * 3], np.uint8).reshape(-1, 3).astype(np.int32)
            v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / float(1 << 23)
        elif bits == 32:
            x = np.frombuffer(pcm, "<i4").astype(np.float32) / float(1 << 31)
        else:
            raise AudioFormatError(f"{bits}-bit PCM is not read")
    elif kind == 3:
        x = np.frombuffer(pcm, "<f4" if bits == 32 else "<f8").astype(np.float32)
    else:
        raise AudioFormatError(f"WAV format tag {kind} is not read (PCM and IEEE float are)")
    n = len(x) // channels
    return torch.from_numpy(x[: n * channels].reshape(n, channels).T.copy()), rate


def encode_wav(samples: torch.Tensor, rate: int, bits: int = 16) -> bytes:
    """float ``[channels, n]`` or ``[n]`` in -1..1 -> 16-bit PCM (or 32-bit float with ``bits=32``)."""
    x = samples.detach().cpu().float()
    if x.dim() == 1:
        x = x[None]
    channels, n = x.shape
    inter = x.t().contiguous().numpy()
    if bits == 16:
        body = np.clip(np.rint(inter * 32767.0), -32768, 32767).astype("<i2").tobytes()
        kind = 1
    elif bits == 32:
        body = inter.astype("<f4").tobytes()
        kind = 3
    else:
        raise AudioFormatError("16-bit PCM or 32-bit float")
    block = channels * bits // 8
    fmt = struct.pack("<HHIIHH", kind, channels, rate, rate * block, block, bits)
    return b"RIFF" + struct.pack("<I", 36 + len(body)) + b"WAVE" + b"fmt " + struct.pack("<I", 16) + fmt + \
        b"data" + struct.pack("<I", len(body)) + body


def read_wav(path: str) -> Tuple[torch.Tensor, int]:
    with open(path, "rb") as f:
        return decode_wav(f.read())


def write_wav(path: str, samples: torch.Tensor, rate: int, bits: int = 16) -> None:
    with open(path, "wb") as f:
        f.write(encode_wav(samples, rate, bits))


# ---------------------------------------------------------------------------------------------------------------------
# resampling
# ---------------------------------------------------------------------------------------------------------------------
def decode_audio(data: bytes) -> Tuple[torch.Tensor, int]:
    """Decode by content: RIFF / WAVE or FLAC. float32 ``[channels, n]`` and the sample rate."""
    if data[:4] == b"RIFF":
        return decode_wav(data)
    if data[:4] == b"fLaC":
        from .flac import decode_flac
        return decode_flac(data)
    raise AudioFormatError("unknown audio format (WAV and FLAC are read)")


def read_audio(path: str) -> Tuple[torch.Tensor, int]:
    with open(path, "rb") as f:
        return decode_audio(f.read())


def resample(x: torch.Tensor, rate_in: int, rate_out: int, zeros: int = 16, rolloff: float = 0.95) -> torch.Tensor:
    """Band-limited polyphase resampling of ``[..., n]`` by the rational factor ``rate_out / rate_in``: a Hann-windowed
    sinc low-pass at ``rolloff`` x the lower Nyquist, one filter phase per output position modulo the up factor, applied
    as a strided convolution."""
    if rate_in == rate_out:
        return x.clone()
    g = math.gcd(rate_in, rate_out)
    up, down = rate_out // g, rate_in // g
    cutoff = rolloff * min(1.0, up / down)                 # relative to the input Nyquist
    half = int(math.ceil(zeros / cutoff))
    shape = x.shape
    v = x.reshape(-1, 1, shape[-1]).float()
    n_out = int(math.ceil(shape[-1] * up / down))
    # output sample j sits at input time j * down / up = q + phase / up; the kernel for that phase spans inputs q-half..q+half
    taps = torch.arange(-half, half + 1, device=x.device, dtype=torch.float64)
    phases = torch.arange(up, device=x.device, dtype=torch.float64) / up
    t = (taps[None] - phases[:, None]) * cutoff
    win = torch.cos(t / (zeros + 1e-9) * math.pi / 2).pow(2) * (t.abs() < zeros)
    kern = (torch.sinc(t) * win * cutoff).float()                             # [up, 2 half + 1]
    padded = torch.nn.functional.pad(v, (half, half + down))
    out = torch.empty(v.shape[0], n_out, device=x.device)
    for p in range(up):
        js = torch.arange(p, n_out, up, device=x.device)                   # outputs with j * down % up == (p * down) % up
        if len(js) == 0:
            continue
        phase = (p * down) % up
        first = (p * down) // up
        y = torch.nn.functional.conv1d(padded[..., first:], kern[phase].view(1, 1, -1), stride=down)[:, 0]
        out[:, js] = y[:, : len(js)]
    return out.reshape(*shape[:-1], n_out).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------------
# STFT and mel features
# ---------------------------------------------------------------------------------------------------------------------
def stft(x: torch.Tensor, n_fft: int, hop: int, window: Optional[torch.Tensor] = None, center: bool = True) -> torch.Tensor:
    """Complex spectrogram ``[..., n_fft // 2 + 1, frames]`` (Hann window, reflect padding when centred)."""
    w = window if window is not None else torch.hann_window(n_fft, device=x.device)
    return torch.stft(x.float(), n_fft, hop, n_fft, w.to(x.device), center=center, pad_mode="reflect", return_complex=True)


def hz_to_mel(f, scale: str = "slaney"):
    f = np.asarray(f, np.float64)
    if scale == "htk":
        return 2595.0 * np.log10(1.0 + f / 700.0)
    lin = f / (200.0 / 3)
    log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
    return np.where(f >= 1000.0, log, lin)


def mel_to_hz(m, scale: str = "slaney"):
    m = np.asarray(m, np.float64)
    if scale == "htk":
        return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))


def mel_filters(rate: int, n_fft: int, n_mels: int, f_min: float = 0.0, f_max: Optional[float] = None,
                scale: str = "slaney", normalise: bool = True) -> torch.Tensor:
    """Triangular filter bank ``[n_mels, n_fft // 2 + 1]``; ``normalise`` gives every filter unit area (Slaney)."""
    f_max = f_max or rate / 2
    freqs = np.linspace(0, rate / 2, n_fft // 2 + 1)
    edges = mel_to_hz(np.linspace(hz_to_mel(f_min, scale), hz_to_mel(f_max, scale), n_mels + 2), scale)
    lower = (freqs[None] - edges[:-2, None]) / np.maximum(edges[1:-1, None] - edges[:-2, None], 1e-10)
    upper = (edges[2:, None] - freqs[None]) / np.maximum(edges[2:, None] - edges[1:-1, None], 1e-10)
    bank = np.maximum(0.0, np.minimum(lower, upper))
    if normalise:
        bank *= (2.0 / (edges[2:] - edges[:-2]))[:, None]
    return torch.from_numpy(bank.astype(np.float32))


@dataclass
class MelSpec:
    rate: int = 16000
    n_fft: int = 400
    hop: int = 160
    n_mels: int = 80
    f_min: float = 0.0
    f_max: Optional[float] = None
    scale: str = "slaney"
    log: str = "whisper"           # whisper: log10, clamp to max - 8, (x + 4) / 4;  db: 10 log10 with a floor;  ln: natural log

    @classmethod
    def whisper(cls, n_mels: int = 80) -> "MelSpec":
        return cls(16000, 400, 160, n_mels)


def log_mel(x: torch.Tensor, spec: MelSpec = MelSpec()) -> torch.Tensor:
    """``[..., n]`` samples -> ``[..., n_mels, frames]`` log-mel features."""
    power = stft(x, spec.n_fft, spec.hop).abs().pow(2)
    if spec.log == "whisper":
        power = power[..., :-1]                                        # the reference front end drops the last frame
    bank = mel_filters(spec.rate, spec.n_fft, spec.n_mels, spec.f_min, spec.f_max, spec.scale).to(power.device)
    mel = bank @ power
    if spec.log == "whisper":
        v = mel.clamp_min(1e-10).log10()
        v = torch.maximum(v, v.amax(dim=(-2, -1), keepdim=True) - 8.0)
        return (v + 4.0) / 4.0
    if spec.log == "db":
        return 10.0 * mel.clamp_min(1e-10).log10()
    return mel.clamp_min(1e-10).log()


# ---------------------------------------------------------------------------------------------------------------------
# CTC decoding
# ---------------------------------------------------------------------------------------------------------------------
def ctc_greedy(log_probabilities: torch.Tensor, blank: int = 0, lengths: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Best path, repeats merged, blanks dropped. ``[N, T, classes]`` -> token lists."""
    best = log_probabilities.argmax(-1).tolist()
    out = []
    for n, row in enumerate(best):
        row = row[: lengths[n]] if lengths is not None else row
        seq, prev = [], blank
        for t in row:
            if t != prev and t != blank:
                seq.append(t)
            prev = t
        out.append(seq)
    return out


def ctc_beam(log_probabilities: torch.Tensor, beam: int = 8, blank: int = 0) -> Tuple[List[int], float]:
    """Prefix beam search over one utterance ``[T, classes]``: sums the probability of every alignment of a prefix
    (ending in blank / not in blank tracked apart). Returns (tokens, log-probability)."""
    lp = log_probabilities.detach().cpu().double().numpy()
    NEG = -np.inf
    beams = {(): (0.0, NEG)}                                    # prefix -> (log p ending in blank, log p ending in non-blank)

    def lse(*v):
        m = max(v)
        return m if m == NEG else m + math.log(sum(math.exp(a - m) for a in v))

    for t in range(lp.shape[0]):
        nxt = {}
        top = np.argsort(lp[t])[::-1][: max(beam, 1) * 2]
        for prefix, (pb, pnb) in beams.items():
            for c in top:
                p = lp[t, c]
                if c == blank:
                    b, nb = nxt.get(prefix, (NEG, NEG))
                    nxt[prefix] = (lse(b, pb + p, pnb + p), nb)
                    continue
                new = prefix + (int(c),)
                b, nb = nxt.get(new, (NEG, NEG))
                if prefix and prefix[-1] == c:
                    nxt[new] = (b, lse(nb, pb + p))             # a repeat needs a blank in between
                    sb, snb = nxt.get(prefix, (NEG, NEG))
                    nxt[prefix] = (sb, lse(snb, pnb + p))       # ... otherwise it extends the same prefix
                else:
                    nxt[new] = (b, lse(nb, pb + p, pnb + p))
        beams = dict(sorted(nxt.items(), key=lambda kv: -lse(*kv[1]))[:beam])
    best, (pb, pnb) = max(beams.items(), key=lambda kv: lse(*kv[1]))
    return list(best), lse(pb, pnb)
