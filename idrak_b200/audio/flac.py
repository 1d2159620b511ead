"""FLAC: a decoder for the whole subset of the format encoders produce (constant, verbatim, fixed and LPC subframes,
Rice and escaped residual partitions, wasted bits, independent / left-side / right-side / mid-side stereo, 8 to 32 bits
per sample, fixed and variable block sizes, header CRC-8 and frame CRC-16 checked) and a small encoder (fixed predictors
of order 0 to 4 chosen per block and channel, one Rice parameter per partition, mid-side stereo when it is cheaper) so
that lossless files can be written and round trips tested without another library.

    samples, rate = decode_flac(open("a.flac", "rb").read())      # float32 [channels, n] in [-1, 1)
    data = encode_flac(samples, rate, bits=16)

Reference: the FLAC reader among the reference's audio codecs (src/Idrak.Audio/Codecs).
"""
from __future__ import annotations

import hashlib
import struct
from typing import List, Tuple

import numpy as np
import torch

from . import AudioFormatError

_BLOCK_SIZES = {1: 192, 2: 576, 3: 1152, 4: 2304, 5: 4608, 8: 256, 9: 512, 10: 1024, 11: 2048, 12: 4096, 13: 8192,
                14: 16384, 15: 32768}
_SAMPLE_RATES = {1: 88200, 2: 176400, 3: 192000, 4: 8000, 5: 16000, 6: 22050, 7: 24000, 8: 32000, 9: 44100, 10: 48000, 11: 96000}
_SAMPLE_SIZES = {1: 8, 2: 12, 4: 16, 5: 20, 6: 24, 7: 32}


def _crc_table(poly: int, bits: int) -> List[int]:
    top, mask = 1 << (bits - 1), (1 << bits) - 1
    table = []
    for b in range(256):
        c = b << (bits - 8)
        for _ in range(8):
            c = ((c << 1) ^ poly) & mask if c & top else (c << 1) & mask
        table.append(c)
    return table


_CRC8, _CRC16 = _crc_table(0x07, 8), _crc_table(0x8005, 16)


def crc8(data: bytes) -> int:
    c = 0
    for b in data:
        c = _CRC8[c ^ b]
    return c


def crc16(data: bytes) -> int:
    c = 0
    for b in data:
        c = ((c << 8) & 0xFFFF) ^ _CRC16[(c >> 8) ^ b]
    return c


class _Reader:
    def __init__(self, data: bytes, at: int = 0):
        self.data, self.at, self.acc, self.n = data, at, 0, 0

    def bits(self, count: int) -> int:
        while self.n < count:
            if self.at >= len(self.data):
                raise AudioFormatError("FLAC data ends inside a frame")
            self.acc = (self.acc << 8) | self.data[self.at]
            self.at += 1
            self.n += 8
        self.n -= count
        v = (self.acc >> self.n) & ((1 << count) - 1)
        self.acc &= (1 << self.n) - 1
        return v

    def signed(self, count: int) -> int:
        v = self.bits(count)
        return v - (1 << count) if v >> (count - 1) else v

    def unary(self) -> int:
        """Zeros up to the next one bit."""
        q = 0
        while True:
            if self.n == 0:
                if self.at >= len(self.data):
                    raise AudioFormatError("FLAC data ends inside a frame")
                self.acc, self.n = self.data[self.at], 8
                self.at += 1
            if self.acc == 0:
                q += self.n
                self.n = 0
                continue
            lead = self.n - self.acc.bit_length()
            q += lead
            self.n -= lead + 1
            self.acc &= (1 << self.n) - 1
            return q

    def align(self) -> None:
        self.acc = self.n = 0

    @property
    def byte_position(self) -> int:
        return self.at - self.n // 8


def _residual(r: _Reader, block: int, order: int) -> List[int]:
    method = r.bits(2)
    if method > 1:
        raise AudioFormatError("reserved residual coding method")
    pbits, escape = (4, 15) if method == 0 else (5, 31)
    porder = r.bits(4)
    parts = 1 << porder
    out: List[int] = []
    for p in range(parts):
        count = (block >> porder) - (order if p == 0 else 0)
        if count < 0:
            raise AudioFormatError("residual partition smaller than the predictor order")
        k = r.bits(pbits)
        if k == escape:
            raw = r.bits(5)
            out.extend(r.signed(raw) if raw else 0 for _ in range(count))
            continue
        for _ in range(count):
            u = (r.unary() << k) | (r.bits(k) if k else 0)
            out.append((u >> 1) ^ -(u & 1))
    return out


_FIXED = {0: (), 1: (1,), 2: (2, -1), 3: (3, -3, 1), 4: (4, -6, 4, -1)}


def _subframe(r: _Reader, block: int, bps: int) -> np.ndarray:
    if r.bits(1):
        raise AudioFormatError("subframe padding bit is set")
    kind = r.bits(6)
    wasted = 0
    if r.bits(1):
        wasted = r.unary() + 1
        bps -= wasted
    if kind == 0:
        out = np.full(block, r.signed(bps), dtype=np.int64)
    elif kind == 1:
        out = np.array([r.signed(bps) for _ in range(block)], dtype=np.int64)
    elif 8 <= kind <= 12 or kind >= 32:
        if kind >= 32:
            order = (kind & 31) + 1
            warm = [r.signed(bps) for _ in range(order)]
            precision = r.bits(4) + 1
            if precision == 16:
                raise AudioFormatError("reserved LPC precision")
            shift = r.signed(5)
            if shift < 0:
                raise AudioFormatError("negative LPC shift")
            coefs = [r.signed(precision) for _ in range(order)]
        else:
            order = kind - 8
            warm = [r.signed(bps) for _ in range(order)]
            coefs, shift = list(_FIXED[order]), 0
        res = _residual(r, block, order)
        s = warm + [0] * (block - order)
        for i in range(order, block):
            acc = 0
            for j, c in enumerate(coefs):
                acc += c * s[i - 1 - j]
            s[i] = res[i - order] + (acc >> shift)
        out = np.array(s, dtype=np.int64)
    else:
        raise AudioFormatError(f"reserved subframe type {kind}")
    return out << wasted if wasted else out


def _utf8_number(r: _Reader) -> int:
    first = r.bits(8)
    if first < 0x80:
        return first
    n = 8 - (first ^ 0xFF).bit_length() if first != 0xFF else 8
    if n < 2 or n > 7:
        raise AudioFormatError("bad frame number")
    v = first & ((1 << (7 - n)) - 1)
    for _ in range(n - 1):
        b = r.bits(8)
        if b >> 6 != 2:
            raise AudioFormatError("bad frame number")
        v = (v << 6) | (b & 0x3F)
    return v


def decode_flac_int(data: bytes, verify: bool = True) -> Tuple[np.ndarray, int, int]:
    """Samples as int64 ``[channels, n]``, the sample rate and the bits per sample."""
    if data[:4] != b"fLaC":
        raise AudioFormatError("not a FLAC stream (no fLaC marker)")
    at, info = 4, None
    while True:
        if at + 4 > len(data):
            raise AudioFormatError("FLAC metadata runs past the end of the data")
        head, length = data[at], int.from_bytes(data[at + 1:at + 4], "big")
        body = data[at + 4:at + 4 + length]
        if head & 0x7F == 0:
            if length != 34:
                raise AudioFormatError("STREAMINFO must be 34 bytes")
            packed = int.from_bytes(body[10:18], "big")
            info = {"rate": packed >> 44, "channels": ((packed >> 41) & 7) + 1, "bits": ((packed >> 36) & 31) + 1,
                    "total": packed & ((1 << 36) - 1), "md5": body[18:34]}
        at += 4 + length
        if head & 0x80:
            break
    if info is None:
        raise AudioFormatError("FLAC stream without STREAMINFO")
    chans: List[List[np.ndarray]] = [[] for _ in range(info["channels"])]
    while at + 2 <= len(data):
        if data[at] != 0xFF or data[at + 1] & 0xFE != 0xF8:
            raise AudioFormatError(f"lost frame synchronisation at byte {at}")
        start = at
        r = _Reader(data, at)
        r.bits(16)
        bs_code, sr_code = r.bits(4), r.bits(4)
        assignment, ss_code = r.bits(4), r.bits(3)
        if r.bits(1) or bs_code == 0 or sr_code == 15 or ss_code == 3:
            raise AudioFormatError("reserved value in a frame header")
        _utf8_number(r)
        block = r.bits(8) + 1 if bs_code == 6 else r.bits(16) + 1 if bs_code == 7 else _BLOCK_SIZES[bs_code]
        if sr_code == 12:
            r.bits(8)
        elif sr_code in (13, 14):
            r.bits(16)
        header_end = r.byte_position
        if r.bits(8) != crc8(data[start:header_end]):
            raise AudioFormatError("frame header CRC mismatch")
        bps = info["bits"] if ss_code == 0 else _SAMPLE_SIZES[ss_code]
        if assignment < 8:
            if assignment + 1 != info["channels"]:
                raise AudioFormatError("channel count changes inside the stream")
            subs = [_subframe(r, block, bps) for _ in range(assignment + 1)]
        elif assignment <= 10:
            if info["channels"] != 2:
                raise AudioFormatError("stereo decorrelation in a stream that is not stereo")
            a = _subframe(r, block, bps + (1 if assignment == 9 else 0))
            b = _subframe(r, block, bps + (0 if assignment == 9 else 1))
            if assignment == 8:
                subs = [a, a - b]
            elif assignment == 9:
                subs = [a + b, b]
            else:
                mid = (a << 1) | (b & 1)
                subs = [(mid + b) >> 1, (mid - b) >> 1]
        else:
            raise AudioFormatError("reserved channel assignment")
        r.align()
        end = r.byte_position
        if verify and int.from_bytes(data[end:end + 2], "big") != crc16(data[start:end]):
            raise AudioFormatError("frame CRC mismatch")
        at = end + 2
        for c, s in zip(chans, subs):
            c.append(s)
    out = np.stack([np.concatenate(c) if c else np.zeros(0, np.int64) for c in chans])
    if info["total"]:
        out = out[:, : info["total"]]
    if verify and info["md5"] != bytes(16) and _md5_of(out, info["bits"]) != info["md5"]:
        raise AudioFormatError("decoded samples do not match the stream's MD5 signature")
    return out, info["rate"], info["bits"]


def _md5_of(x: np.ndarray, bits: int) -> bytes:
    """The signature STREAMINFO carries: MD5 of the interleaved samples, little-endian, whole bytes per sample."""
    width = (bits + 7) // 8
    flat = x.T.reshape(-1)
    if width in (1, 2, 4):
        raw = flat.astype({1: "<i1", 2: "<i2", 4: "<i4"}[width]).tobytes()
    else:                                                       # 3-byte samples: the low three bytes of a 32-bit word
        raw = flat.astype("<i4").view(np.uint8).reshape(-1, 4)[:, :3].tobytes()
    return hashlib.md5(raw).digest()


def decode_flac(data: bytes) -> Tuple[torch.Tensor, int]:
    """float32 ``[channels, n]`` in [-1, 1) and the sample rate."""
    ints, rate, bits = decode_flac_int(data)
    return torch.from_numpy((ints / float(1 << (bits - 1))).astype(np.float32)), rate


def read_flac(path: str) -> Tuple[torch.Tensor, int]:
    with open(path, "rb") as f:
        return decode_flac(f.read())


# ---------------------------------------------------------------------------------------------------------------------
# encoder
# ---------------------------------------------------------------------------------------------------------------------
class _Writer:
    def __init__(self):
        self.out = bytearray()
        self.acc = self.n = 0

    def bits(self, value: int, count: int) -> None:
        if count == 0:
            return
        self.acc = (self.acc << count) | (value & ((1 << count) - 1))
        self.n += count
        while self.n >= 8:
            self.n -= 8
            self.out.append((self.acc >> self.n) & 0xFF)
        self.acc &= (1 << self.n) - 1

    def unary(self, q: int) -> None:
        while q >= 32:
            self.bits(0, 32)
            q -= 32
        self.bits(1, q + 1)

    def align(self) -> None:
        if self.n:
            self.bits(0, 8 - self.n)


def _utf8_like(v: int) -> List[int]:
    """The variable-length number of a frame header: UTF-8's scheme extended to 36 bits."""
    if v < 0x80:
        return [v]
    tail = []
    n = 1
    while True:
        tail.append(0x80 | (v & 0x3F))
        v >>= 6
        n += 1
        if v < (1 << (7 - n)):
            break
    return [((0xFF << (8 - n)) & 0xFF) | v] + tail[::-1]


def _rice_bits(u: np.ndarray, k: int) -> int:
    return int((u >> k).sum()) + len(u) * (k + 1)


def _encode_subframe(w: _Writer, s: np.ndarray, bps: int) -> None:
    if len(s) and (s == s[0]).all():
        w.bits(0, 8)                                            # constant
        w.bits(int(s[0]), bps)
        return
    best = None
    for order in range(0, min(4, len(s) - 1) + 1):
        res = s.copy()
        for _ in range(order):
            res = np.diff(res)                                   # residual of the fixed predictor of this order
        res = s[order:] if order == 0 else res
        u = np.where(res >= 0, res << 1, ((-res) << 1) - 1).astype(np.int64)
        k = max(0, int(np.log2(max(u.mean(), 1.0))))
        cost, kk = min((_rice_bits(u, c), c) for c in range(max(0, k - 1), min(k + 2, 30) + 1))
        cost += order * bps
        if best is None or cost < best[0]:
            best = (cost, order, u, kk)
    cost, order, u, k = best
    if cost >= len(s) * bps or k > 30:
        w.bits(1 << 1, 8)                                       # verbatim
        for v in s:
            w.bits(int(v), bps)
        return
    w.bits((8 + order) << 1, 8)
    for v in s[:order]:
        w.bits(int(v), bps)
    w.bits(1 if k > 14 else 0, 2)
    w.bits(0, 4)                                                # one partition
    w.bits(k, 5 if k > 14 else 4)
    mask = (1 << k) - 1
    for v in u.tolist():
        w.unary(v >> k)
        w.bits(v & mask, k)


def encode_flac(samples, rate: int, bits: int = 16, block: int = 4096) -> bytes:
    """Lossless FLAC of ``samples``: float ``[channels, n]`` / ``[n]`` in [-1, 1) (rounded to ``bits``) or an integer
    array already in that range."""
    x = samples.detach().cpu().numpy() if torch.is_tensor(samples) else np.asarray(samples)
    if x.ndim == 1:
        x = x[None]
    if np.issubdtype(x.dtype, np.floating):
        x = np.clip(np.rint(x * (1 << (bits - 1))), -(1 << (bits - 1)), (1 << (bits - 1)) - 1)
    x = x.astype(np.int64)
    channels, n = x.shape
    if not 1 <= channels <= 8 or bits not in (8, 12, 16, 20, 24) or not 0 < rate < (1 << 20):
        raise AudioFormatError("encode_flac writes 1 to 8 channels of 8, 12, 16, 20 or 24 bits")
    ss_code = {8: 1, 12: 2, 16: 4, 20: 5, 24: 6}[bits]
    frames = bytearray()
    sizes = []
    for index, at in enumerate(range(0, n, block)):
        part = x[:, at:at + block]
        size = part.shape[1]
        w = _Writer()
        w.bits(0xFFF8, 16)                                      # sync, fixed block size
        w.bits(7, 4)                                            # block size follows as 16 bits
        w.bits(0, 4)                                            # sample rate: from STREAMINFO
        plans = [(channels - 1, [(part[c], bits) for c in range(channels)])]
        if channels == 2:
            side = part[0] - part[1]
            plans.append((10, [((part[0] + part[1]) >> 1, bits), (side, bits + 1)]))
            plans.append((8, [(part[0], bits), (side, bits + 1)]))
        tried = []
        for assignment, subs in plans:
            t = _Writer()
            for s, b in subs:
                _encode_subframe(t, s, b)
            tried.append((len(t.out) * 8 + t.n, assignment, subs))
        _, assignment, subs = min(tried, key=lambda v: v[0])
        w.bits(assignment, 4)
        w.bits(ss_code, 3)
        w.bits(0, 1)
        for b in _utf8_like(index):                             # the frame number, coded like UTF-8
            w.bits(b, 8)
        w.bits(size - 1, 16)
        w.bits(crc8(bytes(w.out)), 8)
        for s, b in subs:
            _encode_subframe(w, s, b)
        w.align()
        body = bytes(w.out)
        frames += body + struct.pack(">H", crc16(body))
        sizes.append(len(body) + 2)
    md5 = _md5_of(x, bits)
    packed = (rate << 44) | ((channels - 1) << 41) | ((bits - 1) << 36) | n
    info = struct.pack(">HH", min(block, max(n, 16)), min(block, max(n, 16))) + min(sizes or [0]).to_bytes(3, "big") + \
        max(sizes or [0]).to_bytes(3, "big") + packed.to_bytes(8, "big") + md5
    return b"fLaC" + bytes([0x80]) + len(info).to_bytes(3, "big") + info + bytes(frames)


def write_flac(path: str, samples, rate: int, bits: int = 16) -> None:
    with open(path, "wb") as f:
        f.write(encode_flac(samples, rate, bits))
