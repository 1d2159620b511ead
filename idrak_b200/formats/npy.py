"""``.npy`` / ``.npz`` files read and written without numpy's own reader: header parsing, C and Fortran order,
little- and big-endian numbers, format versions 1 to 3.

Reference: NpyFile (src/Idrak.Abstraction/Formats/NpyFile.cs).
"""
from __future__ import annotations

import ast
import io
import struct
import zipfile
from typing import Dict, Union

import torch

_MAGIC = b"\x93NUMPY"
_TYPES = {"f8": torch.float64, "f4": torch.float32, "f2": torch.float16, "i8": torch.int64, "i4": torch.int32,
          "i2": torch.int16, "i1": torch.int8, "u1": torch.uint8, "b1": torch.bool}
_NAMES = {v: k for k, v in _TYPES.items()}


def _parse_header(f) -> tuple:
    if f.read(6) != _MAGIC:
        raise ValueError("not an .npy file (magic bytes differ)")
    major, _minor = f.read(1)[0], f.read(1)[0]
    if major == 1:
        (n,) = struct.unpack("<H", f.read(2))
    elif major in (2, 3):
        (n,) = struct.unpack("<I", f.read(4))
    else:
        raise ValueError(f".npy format version {major} is not known")
    text = f.read(n).decode("utf-8" if major == 3 else "latin1")
    try:
        meta = ast.literal_eval(text)
    except (ValueError, SyntaxError):
        raise ValueError("the .npy header does not parse")
    descr, fortran, shape = meta["descr"], bool(meta["fortran_order"]), tuple(meta["shape"])
    if not isinstance(descr, str):
        raise ValueError("structured .npy arrays are not supported")
    order, code = descr[0], descr[1:]
    if code not in _TYPES:
        raise ValueError(f".npy element type '{descr}' is not supported")
    return order, _TYPES[code], fortran, shape


def load_npy(source: Union[str, bytes, io.IOBase]) -> torch.Tensor:
    f = open(source, "rb") if isinstance(source, str) else (io.BytesIO(source) if isinstance(source, bytes) else source)
    try:
        order, dtype, fortran, shape = _parse_header(f)
        n = 1
        for s in shape:
            n *= s
        size = torch.empty((), dtype=dtype).element_size()
        raw = f.read(n * size)
        if len(raw) != n * size:
            raise ValueError(f".npy data is cut short: {len(raw)} of {n * size} bytes")
        buf = bytearray(raw)
        if order == ">" and size > 1:                         # big-endian: swap to the host's order
            for i in range(0, len(buf), size):
                buf[i:i + size] = buf[i:i + size][::-1]
        t = torch.frombuffer(buf, dtype=dtype) if n else torch.empty(0, dtype=dtype)
        if fortran and len(shape) > 1:
            return t.reshape(tuple(reversed(shape))).permute(*reversed(range(len(shape)))).contiguous()
        return t.reshape(shape).clone()
    finally:
        if isinstance(source, str):
            f.close()


def save_npy(tensor: torch.Tensor, target: Union[str, io.IOBase, None] = None) -> bytes:
    t = tensor.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        t = t.float()                                            # numpy has no bfloat16
    code = _NAMES.get(t.dtype)
    if code is None:
        raise ValueError(f"{t.dtype} cannot be written to .npy")
    descr = ("|" if t.element_size() == 1 else "<") + code
    shape = "(" + ", ".join(str(s) for s in t.shape) + ("," if t.dim() == 1 else "") + ")"
    header = f"{{'descr': '{descr}', 'fortran_order': False, 'shape': {shape}, }}"
    pad = 64 - (10 + len(header) + 1) % 64
    header = header + " " * (pad % 64) + "\n"
    data = _MAGIC + bytes([1, 0]) + struct.pack("<H", len(header)) + header.encode("latin1")
    data += t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
    if isinstance(target, str):
        with open(target, "wb") as f:
            f.write(data)
    elif target is not None:
        target.write(data)
    return data


def load_npz(path: str) -> Dict[str, torch.Tensor]:
    out = {}
    with zipfile.ZipFile(path) as z:
        for name in z.namelist():
            if name.endswith(".npy"):
                out[name[:-4]] = load_npy(z.read(name))
    return out


def save_npz(tensors: Dict[str, torch.Tensor], path: str, compress: bool = False) -> None:
    with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED if compress else zipfile.ZIP_STORED) as z:
        for name, t in tensors.items():
            z.writestr(name + ".npy", save_npy(t))
