"""Baseline JPEG decoder (sequential DCT, Huffman coding, 8-bit samples): grey and YCbCr images with any sampling
factors up to 2 x 2 (4:4:4, 4:2:2, 4:2:0), restart intervals, JFIF / Adobe colour handling. NumPy only.

    pixels = decode_jpeg(open("photo.jpg", "rb").read())        # uint8 [H, W] or [H, W, 3]

Blocks are entropy-decoded in Python, then de-quantised and inverse-transformed for the whole image at once (a
matrix product per axis). Chroma planes are upsampled by replication, so sub-sampled images differ slightly from
decoders that interpolate chroma; 4:4:4 and grey images agree with libjpeg to within rounding of the inverse DCT.
Progressive, arithmetic-coded, 12-bit and CMYK files are refused by name.

Reference: the JPEG reader among the reference's codecs (src/Idrak.Imaging/Codecs).
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np

from .codecs import ImageFormatError

ZIGZAG = np.array([0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6, 7, 14, 21,
                   28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61,
                   54, 47, 55, 62, 63])


def _idct_matrix() -> np.ndarray:
    k = np.arange(8)
    m = np.cos((2 * k[None] + 1) * k[:, None] * np.pi / 16) * 0.5
    m[0] *= 1 / np.sqrt(2)
    return m                                     # rows: frequency, columns: sample


class _Huffman:
    """Canonical code table: ``lookup[(length, code)] = symbol``, decoded bit by bit with a first-code shortcut."""

    def __init__(self, counts: bytes, symbols: bytes):
        self.min_code = [0] * 17
        self.max_code = [-1] * 17
        self.first_index = [0] * 17
        self.symbols = list(symbols)
        code = index = 0
        for length in range(1, 17):
            n = counts[length - 1]
            self.min_code[length] = code
            self.first_index[length] = index
            if n:
                self.max_code[length] = code + n - 1
            code = (code + n) << 1
            index += n


class _Bits:
    def __init__(self, data: bytes, at: int):
        self.data, self.at = data, at
        self.acc = self.n = 0
        self.marker = 0

    def _fill(self):
        while self.n <= 24:
            if self.marker:
                b = 0
            else:
                b = self.data[self.at] if self.at < len(self.data) else 0
                self.at += 1
                if b == 0xFF:
                    nxt = self.data[self.at] if self.at < len(self.data) else 0xD9
                    if nxt == 0:
                        self.at += 1                      # a stuffed zero after a literal FF
                    else:
                        self.marker = nxt                 # a marker ends the entropy-coded segment
                        self.at -= 1
                        b = 0
            self.acc = ((self.acc << 8) | b) & 0xFFFFFFFFFF
            self.n += 8

    def bit(self) -> int:
        if self.n == 0:
            self._fill()
        self.n -= 1
        return (self.acc >> self.n) & 1

    def bits(self, count: int) -> int:
        if count == 0:
            return 0
        if self.n < count:
            self._fill()
        self.n -= count
        return (self.acc >> self.n) & ((1 << count) - 1)

    def symbol(self, h: _Huffman) -> int:
        code = 0
        for length in range(1, 17):
            code = (code << 1) | self.bit()
            if h.max_code[length] >= code >= h.min_code[length] and h.max_code[length] >= 0:
                return h.symbols[h.first_index[length] + code - h.min_code[length]]
        raise ImageFormatError("bad Huffman code in the JPEG scan")

    def restart(self):
        """Drop the remaining bits and step over an RSTn marker."""
        self.acc = self.n = 0
        if self.marker and 0xD0 <= self.marker <= 0xD7:
            self.at += 2
            self.marker = 0
        else:                                            # look for the marker in the byte stream
            while self.at + 1 < len(self.data) and not (self.data[self.at] == 0xFF and 0xD0 <= self.data[self.at + 1] <= 0xD7):
                self.at += 1
            self.at += 2
            self.marker = 0


def _extend(v: int, size: int) -> int:
    return v if v >= (1 << (size - 1)) else v - (1 << size) + 1


def decode_jpeg(data: bytes) -> np.ndarray:
    if data[:2] != b"\xFF\xD8":
        raise ImageFormatError("not a JPEG file")
    at = 2
    quant: Dict[int, np.ndarray] = {}
    huff: Dict[Tuple[int, int], _Huffman] = {}
    frame = None
    restart_interval = 0
    adobe_transform = None
    while at + 4 <= len(data):
        if data[at] != 0xFF:
            at += 1
            continue
        marker = data[at + 1]
        if marker in (0xD8, 0x01) or 0xD0 <= marker <= 0xD7 or marker == 0xFF:
            at += 2 if marker != 0xFF else 1
            continue
        if marker == 0xD9:
            break
        length = struct.unpack(">H", data[at + 2: at + 4])[0]
        body = data[at + 4: at + 2 + length]
        if marker == 0xDB:
            i = 0
            while i < len(body):
                pq, tq = body[i] >> 4, body[i] & 15
                i += 1
                if pq:
                    vals = np.frombuffer(body, ">u2", 64, i).astype(np.int32)
                    i += 128
                else:
                    vals = np.frombuffer(body, np.uint8, 64, i).astype(np.int32)
                    i += 64
                table = np.zeros(64, np.int32)
                table[ZIGZAG] = vals
                quant[tq] = table
        elif marker == 0xC4:
            i = 0
            while i < len(body):
                tc, th = body[i] >> 4, body[i] & 15
                counts = body[i + 1: i + 17]
                total = sum(counts)
                huff[(tc, th)] = _Huffman(counts, body[i + 17: i + 17 + total])
                i += 17 + total
        elif marker in (0xC0, 0xC1):
            precision, H, W, n = struct.unpack(">BHHB", body[:6])
            if precision != 8:
                raise ImageFormatError(f"{precision}-bit JPEG samples are not read")
            comps = [(body[6 + 3 * c], body[7 + 3 * c] >> 4, body[7 + 3 * c] & 15, body[8 + 3 * c]) for c in range(n)]
            frame = (H, W, comps)
        elif marker == 0xC2:
            raise ImageFormatError("progressive JPEG files are not read (baseline only)")
        elif marker in (0xC3, 0xC5, 0xC6, 0xC7, 0xC9, 0xCA, 0xCB, 0xCD, 0xCE, 0xCF):
            raise ImageFormatError("lossless / hierarchical / arithmetic-coded JPEG files are not read")
        elif marker == 0xDD:
            restart_interval = struct.unpack(">H", body[:2])[0]
        elif marker == 0xEE and body[:5] == b"Adobe":
            adobe_transform = body[11]
        elif marker == 0xDA:
            if frame is None:
                raise ImageFormatError("JPEG scan before the frame header")
            n = body[0]
            scan = [(body[1 + 2 * c], body[2 + 2 * c] >> 4, body[2 + 2 * c] & 15) for c in range(n)]
            return _decode_scan(data, at + 2 + length, frame, scan, quant, huff, restart_interval, adobe_transform)
        at += 2 + length
    raise ImageFormatError("JPEG without image data")


def _decode_scan(data, at, frame, scan, quant, huff, restart_interval, adobe_transform) -> np.ndarray:
    H, W, comps = frame
    if len(comps) not in (1, 3):
        raise ImageFormatError(f"{len(comps)}-component JPEG files are not read (grey and YCbCr / RGB are)")
    if len(scan) != len(comps):
        raise ImageFormatError("multi-scan baseline JPEG files are not read")
    hmax, vmax = max(c[1] for c in comps), max(c[2] for c in comps)
    mcux, mcuy = (W + 8 * hmax - 1) // (8 * hmax), (H + 8 * vmax - 1) // (8 * vmax)
    tables = {cid: (td, ta) for cid, td, ta in scan}
    coefs = [np.zeros((mcuy * v, mcux * h, 64), np.int32) for _, h, v, _ in comps]
    bits = _Bits(data, at)
    pred = [0] * len(comps)
    count = 0
    for my in range(mcuy):
        for mx in range(mcux):
            if restart_interval and count and count % restart_interval == 0:
                bits.restart()
                pred = [0] * len(comps)
            count += 1
            for ci, (cid, h, v, tq) in enumerate(comps):
                dc_t, ac_t = huff[(0, tables[cid][0])], huff[(1, tables[cid][1])]
                for by in range(v):
                    for bx in range(h):
                        block = coefs[ci][my * v + by, mx * h + bx]
                        s = bits.symbol(dc_t)
                        pred[ci] += _extend(bits.bits(s), s) if s else 0
                        block[0] = pred[ci]
                        k = 1
                        while k < 64:
                            rs = bits.symbol(ac_t)
                            r, s = rs >> 4, rs & 15
                            if s == 0:
                                if r != 15:
                                    break
                                k += 16
                                continue
                            k += r
                            if k > 63:
                                raise ImageFormatError("JPEG coefficient index out of range")
                            block[ZIGZAG[k]] = _extend(bits.bits(s), s)
                            k += 1
    m = _idct_matrix()
    planes = []
    for ci, (cid, h, v, tq) in enumerate(comps):
        c = (coefs[ci] * quant[tq][None, None]).reshape(mcuy * v, mcux * h, 8, 8).astype(np.float64)
        px = np.einsum("ux,abuv,vy->abxy", m, c, m)              # inverse DCT along both axes
        px = px.transpose(0, 2, 1, 3).reshape(mcuy * v * 8, mcux * h * 8) + 128.0
        if h != hmax or v != vmax:
            px = np.repeat(np.repeat(px, vmax // v, axis=0), hmax // h, axis=1)
        planes.append(px[:H, :W])
    if len(planes) == 1:
        return np.clip(np.rint(planes[0]), 0, 255).astype(np.uint8)
    y, cb, cr = planes
    ids = [c[0] for c in comps]
    is_rgb = adobe_transform == 0 or ids == [ord("R"), ord("G"), ord("B")]
    if is_rgb:
        rgb = np.stack([y, cb, cr], -1)
    else:
        cb, cr = cb - 128.0, cr - 128.0
        rgb = np.stack([y + 1.402 * cr, y - 0.344136 * cb - 0.714136 * cr, y + 1.772 * cb], -1)
    return np.clip(np.rint(rgb), 0, 255).astype(np.uint8)
