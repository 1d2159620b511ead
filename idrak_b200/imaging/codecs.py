"""Image file codecs without external libraries: PNG (8-bit grey, grey + alpha, RGB, RGBA and palette images, all five
row filters, non-interlaced), BMP (uncompressed 8 / 24 / 32-bit) and Netpbm (P2 / P3 / P5 / P6). Images are NumPy
arrays ``[H, W]`` or ``[H, W, C]`` of uint8.

    pixels = decode(open("page.png", "rb").read())
    open("out.png", "wb").write(encode_png(pixels))

Reference: the reference's codecs (src/Idrak.Imaging/Codecs: PNG, JPEG, BMP, Netpbm readers and writers). Baseline JPEG
is read by ``imaging/jpeg.py`` (``decode`` dispatches to it); JPEG is not written.
"""
from __future__ import annotations

import struct
import zlib
from typing import Optional

import numpy as np

PNG_MAGIC = b"\x89PNG\r\n\x1a\n"


class ImageFormatError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------------------------------
# PNG
# ---------------------------------------------------------------------------------------------------------------------
def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def encode_png(pixels: np.ndarray, level: int = 6) -> bytes:
    """uint8 ``[H, W]`` (grey), ``[H, W, 2]`` (grey + alpha), ``[H, W, 3]`` (RGB) or ``[H, W, 4]`` (RGBA). Rows are
    written with the filter (none / sub / up / average / Paeth) whose residual has the smallest absolute sum."""
    a = np.ascontiguousarray(pixels)
    if a.dtype != np.uint8 or a.ndim not in (2, 3):
        raise ImageFormatError("encode_png takes uint8 [H, W] or [H, W, C]")
    if a.ndim == 2:
        a = a[..., None]
    H, W, Cn = a.shape
    colour = {1: 0, 2: 4, 3: 2, 4: 6}.get(Cn)
    if colour is None:
        raise ImageFormatError("1 to 4 channels")
    rows = a.reshape(H, W * Cn).astype(np.int16)
    prev = np.zeros(W * Cn, np.int16)
    raw = bytearray()
    for y in range(H):
        cur = rows[y]
        left = np.concatenate([np.zeros(Cn, np.int16), cur[:-Cn]])
        upleft = np.concatenate([np.zeros(Cn, np.int16), prev[:-Cn]])
        cands = [cur, cur - left, cur - prev, cur - ((left + prev) >> 1), cur - _paeth(left, prev, upleft)]
        best = min(range(5), key=lambda f: int(np.abs(((cands[f] + 128) & 0xFF) - 128).sum()))
        raw.append(best)
        raw += (cands[best] & 0xFF).astype(np.uint8).tobytes()
        prev = cur
    ihdr = struct.pack(">IIBBBBB", W, H, 8, colour, 0, 0, 0)
    return PNG_MAGIC + _chunk(b"IHDR", ihdr) + _chunk(b"IDAT", zlib.compress(bytes(raw), level)) + _chunk(b"IEND", b"")


def _paeth(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    p = a + b - c
    pa, pb, pc = np.abs(p - a), np.abs(p - b), np.abs(p - c)
    return np.where((pa <= pb) & (pa <= pc), a, np.where(pb <= pc, b, c))


def decode_png(data: bytes) -> np.ndarray:
    if data[:8] != PNG_MAGIC:
        raise ImageFormatError("not a PNG file")
    at = 8
    ihdr = None
    idat = bytearray()
    palette: Optional[np.ndarray] = None
    trns: Optional[bytes] = None
    while at + 8 <= len(data):
        length, tag = struct.unpack(">I4s", data[at: at + 8])
        body = data[at + 8: at + 8 + length]
        if len(body) != length:
            raise ImageFormatError("truncated PNG chunk")
        crc = struct.unpack(">I", data[at + 8 + length: at + 12 + length])[0]
        if zlib.crc32(tag + body) & 0xFFFFFFFF != crc:
            raise ImageFormatError(f"bad checksum in chunk {tag.decode('latin-1')}")
        at += 12 + length
        if tag == b"IHDR":
            ihdr = struct.unpack(">IIBBBBB", body)
        elif tag == b"PLTE":
            palette = np.frombuffer(body, np.uint8).reshape(-1, 3)
        elif tag == b"tRNS":
            trns = body
        elif tag == b"IDAT":
            idat += body
        elif tag == b"IEND":
            break
    if ihdr is None:
        raise ImageFormatError("PNG without a header")
    W, H, depth, colour, _, _, interlace = ihdr
    if interlace:
        raise ImageFormatError("interlaced PNG files are not read")
    channels = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}.get(colour)
    if channels is None or depth not in (1, 2, 4, 8, 16) or (depth < 8 and colour not in (0, 3)):
        raise ImageFormatError("unsupported PNG colour type / bit depth")
    bpp = max(1, channels * depth // 8)                  # bytes per complete pixel, the filter's distance
    stride = (W * channels * depth + 7) // 8
    raw = zlib.decompress(bytes(idat))
    if len(raw) < H * (stride + 1):
        raise ImageFormatError("PNG pixel data is too short")
    out = np.zeros((H, stride), np.uint8)
    prev = np.zeros(stride, np.int32)
    for y in range(H):
        f = raw[y * (stride + 1)]
        line = np.frombuffer(raw, np.uint8, stride, y * (stride + 1) + 1).astype(np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 0xFF
        elif f in (1, 3, 4):
            cur = np.zeros(stride, np.int32)
            for i in range(stride):                      # left neighbours depend on decoded values: sequential
                a = cur[i - bpp] if i >= bpp else 0
                b = prev[i]
                if f == 1:
                    pred = a
                elif f == 3:
                    pred = (a + b) >> 1
                else:
                    c = prev[i - bpp] if i >= bpp else 0
                    p = a + b - c
                    pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
                    pred = a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)
                cur[i] = (line[i] + pred) & 0xFF
        else:
            raise ImageFormatError(f"unknown PNG row filter {f}")
        out[y] = cur
        prev = cur
    if depth == 16:
        px = out.reshape(H, W * channels, 2)[..., 0]     # keep the high byte
    elif depth < 8:
        bits = np.unpackbits(out, axis=1)[:, : W * depth].reshape(H, W, depth)
        px = (bits * (1 << np.arange(depth - 1, -1, -1))).sum(-1).astype(np.uint8)
        if colour == 0:
            px = (px.astype(np.int32) * 255 // ((1 << depth) - 1)).astype(np.uint8)
    else:
        px = out
    px = px.reshape(H, W, channels) if depth >= 8 else px.reshape(H, W, 1)
    if colour == 3:
        if palette is None:
            raise ImageFormatError("palette PNG without a palette")
        idx = px[..., 0]
        rgb = palette[np.minimum(idx, len(palette) - 1)]
        if trns is not None:
            alpha = np.full(256, 255, np.uint8)
            alpha[: len(trns)] = np.frombuffer(trns, np.uint8)
            return np.concatenate([rgb, alpha[idx][..., None]], axis=-1)
        return rgb
    return px[..., 0] if channels == 1 else px


# ---------------------------------------------------------------------------------------------------------------------
# BMP
# ---------------------------------------------------------------------------------------------------------------------
def encode_bmp(pixels: np.ndarray) -> bytes:
    """uint8 ``[H, W]`` (written as 8-bit with a grey palette) or ``[H, W, 3]`` RGB (24-bit)."""
    a = np.ascontiguousarray(pixels)
    if a.dtype != np.uint8:
        raise ImageFormatError("encode_bmp takes uint8")
    if a.ndim == 3 and a.shape[2] == 1:
        a = a[..., 0]
    H, W = a.shape[:2]
    if a.ndim == 2:
        bits, palette = 8, b"".join(bytes((i, i, i, 0)) for i in range(256))
        rows = a
    elif a.shape[2] == 3:
        bits, palette = 24, b""
        rows = a[..., ::-1].reshape(H, W * 3)
    else:
        raise ImageFormatError("grey or RGB")
    stride = (rows.shape[1] + 3) // 4 * 4
    body = np.zeros((H, stride), np.uint8)
    body[:, : rows.shape[1]] = rows[::-1]
    offset = 14 + 40 + len(palette)
    header = b"BM" + struct.pack("<IHHI", offset + body.size, 0, 0, offset)
    info = struct.pack("<IiiHHIIiiII", 40, W, H, 1, bits, 0, body.size, 2835, 2835, 256 if bits == 8 else 0, 0)
    return header + info + palette + body.tobytes()


def decode_bmp(data: bytes) -> np.ndarray:
    if data[:2] != b"BM":
        raise ImageFormatError("not a BMP file")
    offset = struct.unpack("<I", data[10:14])[0]
    size = struct.unpack("<I", data[14:18])[0]
    if size < 40:
        raise ImageFormatError("old-style BMP headers are not read")
    W, Hs, _, bits, compression = struct.unpack("<iiHHI", data[18:34])
    if compression not in (0, 3) or bits not in (8, 24, 32):
        raise ImageFormatError("only uncompressed 8 / 24 / 32-bit BMP files are read")
    H, flip = abs(Hs), Hs > 0
    stride = (W * bits // 8 + 3) // 4 * 4
    rows = np.frombuffer(data, np.uint8, H * stride, offset).reshape(H, stride)
    if flip:
        rows = rows[::-1]
    if bits == 8:
        colours = struct.unpack("<I", data[46:50])[0] or 256
        pal = np.frombuffer(data, np.uint8, colours * 4, 14 + size).reshape(-1, 4)[:, 2::-1]
        px = pal[rows[:, :W]]
        return px[..., 0].copy() if (px[..., 0] == px[..., 1]).all() and (px[..., 1] == px[..., 2]).all() else px.copy()
    Cn = bits // 8
    px = rows[:, : W * Cn].reshape(H, W, Cn)
    return np.ascontiguousarray(px[..., 2::-1])          # BGR(A) -> RGB


# ---------------------------------------------------------------------------------------------------------------------
# Netpbm
# ---------------------------------------------------------------------------------------------------------------------
def encode_pnm(pixels: np.ndarray) -> bytes:
    a = np.ascontiguousarray(pixels)
    if a.dtype != np.uint8:
        raise ImageFormatError("encode_pnm takes uint8")
    if a.ndim == 3 and a.shape[2] == 1:
        a = a[..., 0]
    if a.ndim == 2:
        return b"P5\n%d %d\n255\n" % (a.shape[1], a.shape[0]) + a.tobytes()
    if a.ndim == 3 and a.shape[2] == 3:
        return b"P6\n%d %d\n255\n" % (a.shape[1], a.shape[0]) + a.tobytes()
    raise ImageFormatError("grey or RGB")


def decode_pnm(data: bytes) -> np.ndarray:
    magic = data[:2]
    if magic not in (b"P2", b"P3", b"P5", b"P6"):
        raise ImageFormatError("not a Netpbm grey / colour file")
    at = 2
    fields = []
    while len(fields) < 3:
        while at < len(data) and data[at: at + 1].isspace():
            at += 1
        if data[at: at + 1] == b"#":
            while at < len(data) and data[at: at + 1] != b"\n":
                at += 1
            continue
        start = at
        while at < len(data) and not data[at: at + 1].isspace():
            at += 1
        fields.append(int(data[start: at]))
    W, H, maxval = fields
    Cn = 3 if magic in (b"P3", b"P6") else 1
    if magic in (b"P5", b"P6"):
        at += 1                                          # the single whitespace after maxval
        if maxval > 255:
            px = np.frombuffer(data, ">u2", W * H * Cn, at).astype(np.float64)
        else:
            px = np.frombuffer(data, np.uint8, W * H * Cn, at).astype(np.float64)
    else:
        px = np.array(data[at:].split()[: W * H * Cn], np.float64)
    if maxval != 255:
        px = np.rint(px * 255.0 / maxval)
    px = px.astype(np.uint8).reshape(H, W, Cn)
    return px[..., 0] if Cn == 1 else px


# ---------------------------------------------------------------------------------------------------------------------
def decode(data: bytes) -> np.ndarray:
    """Decode by content: PNG, BMP or Netpbm."""
    if data[:8] == PNG_MAGIC:
        return decode_png(data)
    if data[:2] == b"BM":
        return decode_bmp(data)
    if data[:1] == b"P" and data[1:2] in b"2356":
        return decode_pnm(data)
    if data[:2] == b"\xFF\xD8":
        from .jpeg import decode_jpeg
        return decode_jpeg(data)
    raise ImageFormatError("unknown image format (PNG, JPEG, BMP and Netpbm are read)")


def encode(pixels: np.ndarray, format: str) -> bytes:
    f = format.lower().lstrip(".")
    if f == "png":
        return encode_png(pixels)
    if f == "bmp":
        return encode_bmp(pixels)
    if f in ("pnm", "pgm", "ppm"):
        return encode_pnm(pixels)
    if f in ("jpg", "jpeg"):
        from .jpeg import encode_jpeg
        return encode_jpeg(pixels)
    raise ImageFormatError(f"cannot write '{format}' (png, jpeg, bmp, pgm / ppm)")
