import math

import numpy as np
import pytest
import torch

from idrak_b200 import audio as A


def _tone(freq, rate, seconds=1.0, amp=0.5):
    return torch.sin(2 * math.pi * freq * torch.arange(int(rate * seconds)) / rate) * amp


@pytest.mark.parametrize("rate_in,rate_out", [(48000, 16000), (44100, 16000), (16000, 22050), (8000, 16000), (16000, 16000)])
def test_resample_keeps_tones_and_removes_aliases(rate_in, rate_out):
    y = A.resample(_tone(440, rate_in), rate_in, rate_out)
    ref = _tone(440, rate_out)
    assert y.shape == ref.shape
    assert (y[400:-400] - ref[400:-400]).abs().max().item() < 2e-3
    if rate_out < rate_in:                       # a tone above the new Nyquist must not fold back
        hi = A.resample(_tone(0.45 * rate_in, rate_in, amp=1.0), rate_in, rate_out)
        assert hi[500:-500].abs().max().item() < 5e-3
    batch = A.resample(torch.stack([_tone(300, rate_in), _tone(500, rate_in)]), rate_in, rate_out)
    assert batch.shape[0] == 2 and torch.allclose(batch[0], A.resample(_tone(300, rate_in), rate_in, rate_out), atol=1e-6)


def test_wav_round_trips_and_reads_other_sample_formats():
    x = torch.stack([_tone(440, 8000, 0.1), _tone(880, 8000, 0.1)])
    y, rate = A.decode_wav(A.encode_wav(x, 8000))
    assert rate == 8000 and y.shape == x.shape and (y - x).abs().max().item() < 1e-4
    y, _ = A.decode_wav(A.encode_wav(x, 8000, bits=32))
    assert torch.equal(y, x)
    import struct
    def wav(kind, bits, body, channels=1):
        block = channels * bits // 8
        fmt = struct.pack("<HHIIHH", kind, channels, 8000, 8000 * block, block, bits)
        return b"RIFF" + struct.pack("<I", 36 + len(body)) + b"WAVE" + b"fmt " + struct.pack("<I", 16) + fmt + b"LIST" + \
            struct.pack("<I", 3) + b"abc\0" + b"data" + struct.pack("<I", len(body)) + body
    y, _ = A.decode_wav(wav(1, 8, bytes([0, 128, 255])))
    assert torch.allclose(y[0], torch.tensor([-1.0, 0.0, 127 / 128]))
    y, _ = A.decode_wav(wav(1, 24, bytes([0, 0, 0x40, 0, 0, 0xC0])))
    assert torch.allclose(y[0], torch.tensor([0.5, -0.5]))
    y, _ = A.decode_wav(wav(3, 64, np.array([0.25, -0.75]).astype("<f8").tobytes()))
    assert torch.allclose(y[0], torch.tensor([0.25, -0.75]))
    with pytest.raises(A.AudioFormatError):
        A.decode_wav(b"OggS" + bytes(40))
    with pytest.raises(A.AudioFormatError, match="tag 85"):
        A.decode_wav(wav(85, 16, b"\0\0"))


def test_log_mel_equals_the_whisper_front_end():
    transformers = pytest.importorskip("transformers")
    fe = transformers.WhisperFeatureExtractor()
    sig = (torch.randn(16000 * 2, generator=torch.Generator().manual_seed(0)) * 0.1).numpy()
    ref = fe(sig, sampling_rate=16000, return_tensors="np").input_features[0]
    padded = np.zeros(16000 * 30, np.float32)
    padded[: len(sig)] = sig
    got = A.log_mel(torch.from_numpy(padded), A.MelSpec.whisper()).numpy()
    assert got.shape == ref.shape == (80, 3000) and np.abs(ref - got).max() < 1e-4


def test_mel_filters_and_stft():
    bank = A.mel_filters(16000, 400, 80)
    assert bank.shape == (80, 201) and (bank >= 0).all() and (bank.sum(1) > 0).all()
    peaks = bank.argmax(1)
    assert (peaks[1:] >= peaks[:-1]).all()                      # centre frequencies rise
    htk = A.mel_filters(16000, 512, 40, scale="htk", normalise=False)
    assert abs(htk.max().item() - 1.0) < 0.1
    assert np.allclose(A.mel_to_hz(A.hz_to_mel([100.0, 1000.0, 4000.0])), [100.0, 1000.0, 4000.0])
    s = A.stft(_tone(1000, 16000), 400, 160).abs()
    assert s.shape == (201, 101) and int(s[:, 50].argmax()) == 25      # 1000 Hz / (16000 / 400) = bin 25
    db = A.log_mel(_tone(1000, 16000), A.MelSpec(log="db"))
    assert db.shape[0] == 80 and torch.isfinite(db).all()


def test_ctc_decoders():
    # frames: a a - a b b -  ->  a a b
    ids = [1, 1, 0, 1, 2, 2, 0]
    lp = torch.full((1, 7, 3), -10.0)
    for t, c in enumerate(ids):
        lp[0, t, c] = 0.0
    lp = lp.log_softmax(-1)
    assert A.ctc_greedy(lp) == [[1, 1, 2]]
    assert A.ctc_greedy(lp, lengths=[3]) == [[1]]
    seq, score = A.ctc_beam(lp[0], beam=4)
    assert seq == [1, 1, 2] and score < 0
    # a case where the best path differs from the most probable labelling: p(blank) = 0.6 each frame, but the
    # two ways to emit "a" (a-, -a, aa) sum to more than "--"
    lp2 = torch.tensor([[0.6, 0.4], [0.6, 0.4]]).log()
    assert A.ctc_greedy(lp2[None]) == [[]]
    seq, score = A.ctc_beam(lp2, beam=4)
    assert seq == [1] and abs(math.exp(score) - 0.64) < 1e-6
