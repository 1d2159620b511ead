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


# ---------------------------------------------------------------------------------------------------------------------
# encoder
# ---------------------------------------------------------------------------------------------------------------------
_Q_LUMA = np.array([16, 11, 10, 16, 24, 40, 51, 61, 12, 12, 14, 19, 26, 58, 60, 55, 14, 13, 16, 24, 40, 57, 69, 56,
                    14, 17, 22, 29, 51, 87, 80, 62, 18, 22, 37, 56, 68, 109, 103, 77, 24, 35, 55, 64, 81, 104, 113, 92,
                    49, 64, 78, 87, 103, 121, 120, 101, 72, 92, 95, 98, 112, 100, 103, 99]).reshape(8, 8)
_Q_CHROMA = np.array([17, 18, 24, 47, 99, 99, 99, 99, 18, 21, 26, 66, 99, 99, 99, 99, 24, 26, 56, 99, 99, 99, 99, 99,
                      47, 66, 99, 99, 99, 99, 99, 99] + [99] * 32).reshape(8, 8)


def _scaled_table(base: np.ndarray, quality: int) -> np.ndarray:
    """The base table scaled the way the Independent JPEG Group's quality setting does (50 = the table itself)."""
    q = min(max(int(quality), 1), 100)
    scale = 5000 // q if q < 50 else 200 - 2 * q
    return np.clip((base * scale + 50) // 100, 1, 255).astype(np.int32)


def _code_lengths(freq: Dict[int, int]) -> Dict[int, int]:
    """Huffman code lengths of at most 16 bits for the symbols of ``freq`` (no code of all ones: one code point is kept
    free, as the format demands). Plain Huffman merging, then the longest codes are shortened by moving symbols up."""
    import heapq
    items = [(f, i, (s,)) for i, (s, f) in enumerate(sorted(freq.items()))]
    items.append((0, len(items), (-1,)))                       # the reserved code point
    if len(items) == 2:
        return {items[0][2][0]: 1}
    depth = {s: 0 for _, _, (s,) in items}
    heapq.heapify(items)
    tie = len(items)
    while len(items) > 1:
        a = heapq.heappop(items)
        b = heapq.heappop(items)
        for s in a[2] + b[2]:
            depth[s] += 1
        heapq.heappush(items, (a[0] + b[0], tie, a[2] + b[2]))
        tie += 1
    counts = [0] * 64
    for d in depth.values():
        counts[d] += 1
    for length in range(len(counts) - 1, 16, -1):              # the standard's adjustment: pull long codes under 17 bits
        while counts[length] > 0:
            j = length - 2
            while counts[j] == 0:
                j -= 1
            counts[length] -= 2
            counts[length - 1] += 1
            counts[j + 1] += 2
            counts[j] -= 1
    # hand the lengths out again: most frequent symbols get the shortest codes; the reserved point takes the longest
    order = sorted((s for s in depth if s != -1), key=lambda s: (-freq[s], s))
    lengths, at = {}, 0
    pool = [length for length in range(1, 17) for _ in range(counts[length])]
    pool = pool[:-1] if len(pool) > len(order) else pool       # drop the reserved code point's slot
    for s, length in zip(order, pool):
        lengths[s] = length
    return lengths


def _canonical(lengths: Dict[int, int]):
    """(counts per length 1..16, symbols in code order, symbol -> (code, length))."""
    by_len = sorted(lengths.items(), key=lambda kv: (kv[1], kv[0]))
    counts = [0] * 16
    codes, code, prev = {}, 0, 0
    for s, length in by_len:
        code <<= length - prev
        prev = length
        codes[s] = (code, length)
        counts[length - 1] += 1
        code += 1
    return counts, [s for s, _ in by_len], codes


class _BitWriter:
    def __init__(self):
        self.out = bytearray()
        self.acc = self.n = 0

    def put(self, code: int, length: int):
        self.acc = (self.acc << length) | (code & ((1 << length) - 1))
        self.n += length
        while self.n >= 8:
            self.n -= 8
            byte = (self.acc >> self.n) & 0xFF
            self.out.append(byte)
            if byte == 0xFF:
                self.out.append(0)                             # a data byte of all ones is followed by a zero
        self.acc &= (1 << self.n) - 1

    def finish(self) -> bytes:
        if self.n:
            self.put((1 << (8 - self.n)) - 1, 8 - self.n)      # pad with ones
        return bytes(self.out)


def _category(v: int) -> int:
    return int(abs(v)).bit_length()


def _symbols(blocks: np.ndarray):
    """Per component: the (DC symbol, extra bits) and (AC symbol, extra bits) stream of its zig-zagged blocks."""
    dc, ac, prev = [], [], 0
    for block in blocks:
        d = int(block[0]) - prev
        prev = int(block[0])
        c = _category(d)
        dc.append((c, d if d >= 0 else d + (1 << c) - 1, c))
        run = 0
        row = []
        last = int(np.max(np.nonzero(block)[0])) if block[1:].any() else 0
        for k in range(1, last + 1):
            v = int(block[k])
            if v == 0:
                run += 1
                continue
            while run > 15:
                row.append((0xF0, 0, 0))
                run -= 16
            c = _category(v)
            row.append(((run << 4) | c, v if v >= 0 else v + (1 << c) - 1, c))
            run = 0
        if last < 63:
            row.append((0x00, 0, 0))                           # end of block
        ac.append(row)
    return dc, ac


def encode_jpeg(pixels: np.ndarray, quality: int = 90, subsample: bool = False) -> bytes:
    """Baseline JPEG (JFIF) of a uint8 grey ``[H, W]`` or colour ``[H, W, 3]`` image. ``quality`` 1..100 scales the standard
    quantisation tables; ``subsample`` stores the chroma planes at half resolution in both directions (4:2:0). The
    Huffman tables are built from the image's own symbol statistics."""
    px = np.asarray(pixels)
    if px.dtype != np.uint8 or px.ndim not in (2, 3) or (px.ndim == 3 and px.shape[2] not in (1, 3)):
        raise ImageFormatError("encode_jpeg takes uint8 pixels shaped [H, W] or [H, W, 3]")
    if px.ndim == 3 and px.shape[2] == 1:
        px = px[:, :, 0]
    H, W = px.shape[:2]
    if H < 1 or W < 1 or H > 65535 or W > 65535:
        raise ImageFormatError("image size must be 1..65535 in both directions")
    grey = px.ndim == 2
    f = px.astype(np.float64)
    if grey:
        planes = [f]
    else:
        r, g, b = f[..., 0], f[..., 1], f[..., 2]
        planes = [0.299 * r + 0.587 * g + 0.114 * b,
                  -0.168735892 * r - 0.331264108 * g + 0.5 * b + 128.0,
                  0.5 * r - 0.418687589 * g - 0.081312411 * b + 128.0]
    sub = bool(subsample) and not grey
    mcu = 16 if sub else 8
    Hp, Wp = -(-H // mcu) * mcu, -(-W // mcu) * mcu
    planes = [np.pad(p, ((0, Hp - H), (0, Wp - W)), mode="edge") for p in planes]
    if sub:
        planes[1:] = [p.reshape(Hp // 2, 2, Wp // 2, 2).mean((1, 3)) for p in planes[1:]]
    tables = [_scaled_table(_Q_LUMA, quality), _scaled_table(_Q_CHROMA, quality)]
    D = _idct_matrix()                                         # forward transform: D X D^T
    comp_blocks = []
    for ci, p in enumerate(planes):
        h, w = p.shape
        blocks = (p - 128.0).reshape(h // 8, 8, w // 8, 8).transpose(0, 2, 1, 3)          # [by, bx, 8, 8]
        coeff = np.einsum("ui,yxij,vj->yxuv", D, blocks, D)
        q = np.rint(coeff / tables[0 if ci == 0 else 1]).astype(np.int32)
        comp_blocks.append(q.reshape(h // 8, w // 8, 64)[:, :, ZIGZAG])
    # block order of the scan: component by component inside each minimum coded unit
    by, bx = Hp // mcu, Wp // mcu
    order: List[Tuple[int, np.ndarray]] = []
    per_comp: List[List[np.ndarray]] = [[] for _ in planes]
    for y in range(by):
        for x in range(bx):
            if sub:
                for dy in (0, 1):
                    for dx in (0, 1):
                        per_comp[0].append(comp_blocks[0][2 * y + dy, 2 * x + dx])
                        order.append((0, len(per_comp[0]) - 1))
                for ci in (1, 2):
                    per_comp[ci].append(comp_blocks[ci][y, x])
                    order.append((ci, len(per_comp[ci]) - 1))
            else:
                for ci in range(len(planes)):
                    per_comp[ci].append(comp_blocks[ci][y, x])
                    order.append((ci, len(per_comp[ci]) - 1))
    streams = [_symbols(np.stack(blocks)) for blocks in per_comp]
    # statistics -> tables: one DC and one AC table for luma, one pair for chroma
    def table_for(kind: int, comps) -> Dict[int, int]:
        freq: Dict[int, int] = {}
        for ci in comps:
            rows = streams[ci][kind]
            for row in (rows if kind else [rows]):
                for sym, _, _ in row:
                    freq[sym] = freq.get(sym, 0) + 1
        return _code_lengths(freq)
    groups = [(0,)] if grey else [(0,), (1, 2)]
    huff = [[_canonical(table_for(kind, comps)) for kind in (0, 1)] for comps in groups]
    # ---- the file
    out = bytearray(b"\xFF\xD8")
    out += b"\xFF\xE0" + struct.pack(">H5sHBHHBB", 16, b"JFIF\0", 0x0101, 0, 1, 1, 0, 0)
    for ti, t in enumerate(tables[: 1 if grey else 2]):
        out += b"\xFF\xDB" + struct.pack(">HB", 67, ti) + bytes(int(v) for v in t.reshape(64)[ZIGZAG])
    n = len(planes)
    out += b"\xFF\xC0" + struct.pack(">HBHHB", 8 + 3 * n, 8, H, W, n)
    for ci in range(n):
        out += bytes([ci + 1, (0x22 if sub else 0x11) if ci == 0 else 0x11, 0 if ci == 0 else 1])
    for gi, pair in enumerate(huff):
        for kind, (counts, symbols, _) in enumerate(pair):
            out += b"\xFF\xC4" + struct.pack(">HB", 19 + len(symbols), (kind << 4) | gi) + bytes(counts) + bytes(symbols)
    out += b"\xFF\xDA" + struct.pack(">HB", 6 + 2 * n, n)
    for ci in range(n):
        gi = 0 if ci == 0 else 1
        out += bytes([ci + 1, (gi << 4) | gi])
    out += b"\x00\x3F\x00"
    bits = _BitWriter()
    for ci, bi in order:
        gi = 0 if ci == 0 else 1
        dc_codes, ac_codes = huff[gi][0][2], huff[gi][1][2]
        sym, extra, nbits = streams[ci][0][bi]
        bits.put(*dc_codes[sym])
        if nbits:
            bits.put(extra, nbits)
        for sym, extra, nbits in streams[ci][1][bi]:
            bits.put(*ac_codes[sym])
            if nbits:
                bits.put(extra, nbits)
    out += bits.finish() + b"\xFF\xD9"
    return bytes(out)
