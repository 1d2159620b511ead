"""FLAC: lossless round trips through the package's encoder, a hand-built frame that exercises the decoder paths the
encoder never writes (LPC prediction, two Rice partitions, an escaped partition, wasted bits), and the integrity checks."""
import struct

import numpy as np
import pytest
import torch

from idrak_b200.audio import AudioFormatError
from idrak_b200.audio.flac import (_Reader, _utf8_like, _utf8_number, _Writer, crc8, crc16, decode_flac, decode_flac_int,
                                   encode_flac)


def _tone(n=20000, rate=16000, seed=0):
    rng = np.random.default_rng(seed)
    t = np.arange(n) / rate
    return np.stack([0.5 * np.sin(2 * np.pi * 440 * t) + 0.01 * rng.normal(size=n),
                     0.4 * np.sin(2 * np.pi * 445 * t + 0.3) + 0.01 * rng.normal(size=n)])


@pytest.mark.parametrize("bits", [8, 16, 24])
def test_round_trip_is_lossless_and_smaller_than_pcm(bits):
    x = _tone()
    data = encode_flac(x, 16000, bits)
    ints, rate, b = decode_flac_int(data)
    want = np.clip(np.rint(x * (1 << (bits - 1))), -(1 << (bits - 1)), (1 << (bits - 1)) - 1).astype(np.int64)
    assert rate == 16000 and b == bits and np.array_equal(ints, want)
    assert len(data) < 0.85 * x.size * bits / 8
    samples, _ = decode_flac(data)
    assert samples.dtype == torch.float32 and samples.shape == (2, 20000) and samples.abs().max() <= 1.0


def test_silence_constants_noise_and_short_blocks():
    rng = np.random.default_rng(1)
    mono = np.concatenate([np.zeros(5000), rng.normal(size=3000) * 0.9, np.full(2000, 0.25), rng.normal(size=17) * 0.1])
    data = encode_flac(mono, 8000, 16, block=1152)
    ints, rate, _ = decode_flac_int(data)
    assert rate == 8000 and np.array_equal(ints[0], np.clip(np.rint(mono * 32768), -32768, 32767).astype(np.int64))
    assert len(encode_flac(np.zeros(40000), 8000)) < 400                 # constant subframes


def test_frame_numbers_code_like_utf8():
    for v in (0, 127, 128, 2047, 2048, 65535, 65536, (1 << 21) - 1, 1 << 21, (1 << 31) - 1, (1 << 36) - 1):
        assert _utf8_number(_Reader(bytes(_utf8_like(v)))) == v


def _rice(w, values, k):
    for v in values:
        u = (v << 1) if v >= 0 else ((-v) << 1) - 1
        w.unary(u >> k)
        w.bits(u & ((1 << k) - 1), k)


def test_decoder_paths_the_encoder_does_not_write():
    # one mono frame of 16 samples at 16 bits with 2 wasted bits: LPC order 2, coefficients (7, -3) >> 2, two partitions,
    # the second one escaped (raw 6-bit residuals)
    coefs, shift, order, block, wasted = (7, -3), 2, 2, 16, 2
    rng = np.random.default_rng(3)
    res = rng.integers(-9, 10, block - order).tolist()
    s = [100, 104]
    for i in range(order, block):
        s.append(res[i - order] + ((coefs[0] * s[i - 1] + coefs[1] * s[i - 2]) >> shift))
    w = _Writer()
    w.bits(0xFFF8, 16); w.bits(6, 4); w.bits(0, 4); w.bits(0, 4); w.bits(4, 3); w.bits(0, 1)       # 8-bit block size follows
    w.bits(0, 8)                                                                                     # frame number 0
    w.bits(block - 1, 8)
    w.bits(crc8(bytes(w.out)), 8)
    w.bits(0, 1); w.bits(32 + order - 1, 6); w.bits(1, 1); w.unary(wasted - 1)                       # LPC, wasted bits
    for v in s[:order]:
        w.bits(v, 16 - wasted)
    w.bits(5 - 1, 4); w.bits(shift, 5)
    for c in coefs:
        w.bits(c, 5)
    w.bits(0, 2); w.bits(1, 4)                                                                       # Rice, 2 partitions
    w.bits(3, 4); _rice(w, res[: block // 2 - order], 3)
    w.bits(15, 4); w.bits(6, 5)                                                                      # escape: 6 raw bits each
    for v in res[block // 2 - order:]:
        w.bits(v, 6)
    w.align()
    body = bytes(w.out)
    packed = (8000 << 44) | (0 << 41) | (15 << 36) | block
    info = struct.pack(">HH", 16, 16) + bytes(6) + packed.to_bytes(8, "big") + bytes(16)
    data = b"fLaC" + bytes([0x80]) + len(info).to_bytes(3, "big") + info + body + struct.pack(">H", crc16(body))
    ints, rate, bits = decode_flac_int(data)
    assert rate == 8000 and bits == 16 and ints.tolist() == [[v << wasted for v in s]]
    # a flipped bit in the frame is caught by its CRC, a wrong signature by the MD5 check
    broken = bytearray(data)
    broken[-5] ^= 0x10
    with pytest.raises(AudioFormatError, match="CRC"):
        decode_flac_int(bytes(broken))
    good = encode_flac(_tone(3000), 16000)
    tampered = bytearray(good)
    tampered[4 + 4 + 18] ^= 0xFF                                      # first byte of the MD5 in STREAMINFO
    with pytest.raises(AudioFormatError, match="MD5"):
        decode_flac_int(bytes(tampered))
    with pytest.raises(AudioFormatError, match="fLaC"):
        decode_flac_int(b"RIFF" + bytes(40))
