"""GGUF reader: metadata, tensor directory and de-quantisation of ggml block formats to fp32.

Supported tensor types: F32, F16, BF16, F64, I8/I16/I32/I64, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2_K, Q3_K,
Q4_K, Q5_K, Q6_K, Q8_K, IQ4_NL, IQ4_XS. The arithmetic follows ggml's reference de-quantisers operation for
operation in float32, so values are bit-identical to what llama.cpp computes. The codebook ("grid")
types IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S and the ternary TQ1_0 / TQ2_0 are recognised in
the directory (sizes are known, so files holding them open) and raise ``NotImplementedError`` naming the
type when read.

``GgufFile.decoder_spec()`` translates ``<arch>.*`` metadata into a ``DecoderSpec`` and
``GgufFile.idrak_tensors()`` renames ``blk.N.attn_q.weight`` ... into the decoder's checkpoint layout,
undoing the row permutation llama.cpp's converter applies to q/k projections of Llama-family models.

Reference: GgufFile / GgufTypes / GgufModel (src/Idrak/Models/Gguf.cs:31, GgufFile.LowBit.cs, GgufModel.cs).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
QK_K = 256

# type id -> (name, values per block, bytes per block)
TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
    16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50),
    20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82), 23: ("IQ4_XS", 256, 136),
    24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 34: ("TQ1_0", 256, 54), 35: ("TQ2_0", 256, 66),
}
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


@dataclass
class GgufTensorInfo:
    name: str
    shape: Tuple[int, ...]       # outermost first (row-major), i.e. reversed ggml "ne"
    type_id: int
    offset: int                  # absolute file offset

    @property
    def type_name(self) -> str:
        return TYPES[self.type_id][0]

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        _, per, size = TYPES[self.type_id]
        return self.count // per * size


def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.view("<f2").astype(np.float32)


# --------------------------------------------------------------------------- de-quantisers (blocks: [n, bytes])
def _dq_q4_0(b):
    d = _f16(b[:, 0:2].copy())                      # [n,1]
    qs = b[:, 2:18]
    lo = (qs & 0x0F).astype(np.int8) - 8
    hi = (qs >> 4).astype(np.int8) - 8
    return np.concatenate([lo, hi], axis=1).astype(np.float32) * d


def _dq_q4_1(b):
    d, m = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
    qs = b[:, 4:20]
    q = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32)
    return q * d + m


def _q5_high(b_qh):
    qh = b_qh.copy().view("<u4")                                 # [n,1]
    j = np.arange(16, dtype=np.uint32)
    h0 = (((qh >> j) << 4) & 0x10).astype(np.uint8)               # [n,16]
    h1 = ((qh >> (j + 12)) & 0x10).astype(np.uint8)
    return h0, h1


def _dq_q5_0(b):
    d = _f16(b[:, 0:2].copy())
    h0, h1 = _q5_high(b[:, 2:6])
    qs = b[:, 6:22]
    x0 = ((qs & 0x0F) | h0).astype(np.int32) - 16
    x1 = ((qs >> 4) | h1).astype(np.int32) - 16
    return np.concatenate([x0, x1], axis=1).astype(np.float32) * d


def _dq_q5_1(b):
    d, m = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
    h0, h1 = _q5_high(b[:, 4:8])
    qs = b[:, 8:24]
    x0 = ((qs & 0x0F) | h0).astype(np.float32)
    x1 = ((qs >> 4) | h1).astype(np.float32)
    return np.concatenate([x0, x1], axis=1) * d + m


def _dq_q8_0(b):
    d = _f16(b[:, 0:2].copy())
    return b[:, 2:34].view(np.int8).astype(np.float32) * d


def _dq_q8_1(b):
    d = _f16(b[:, 0:2].copy())
    return b[:, 4:36].view(np.int8).astype(np.float32) * d


def _dq_q8_k(b):
    d = b[:, 0:4].copy().view("<f4")
    return b[:, 4:260].view(np.int8).astype(np.float32) * d


def _dq_q2_k(b):
    n = b.shape[0]
    scales, qs = b[:, 0:16], b[:, 16:80]
    d, dmin = _f16(b[:, 80:82].copy()), _f16(b[:, 82:84].copy())
    out = np.empty((n, 256), dtype=np.float32)
    is_ = 0
    for half in range(2):
        q = qs[:, 32 * half: 32 * half + 32]
        for shift in (0, 2, 4, 6):
            for part in range(2):
                sc = scales[:, is_:is_ + 1]
                dl = d * (sc & 0xF).astype(np.float32)
                ml = dmin * (sc >> 4).astype(np.float32)
                v = ((q[:, 16 * part: 16 * part + 16] >> shift) & 3).astype(np.float32)
                y0 = 128 * half + (shift // 2) * 32 + 16 * part
                out[:, y0:y0 + 16] = dl * v - ml
                is_ += 1
    return out


def _dq_q3_k(b):
    n = b.shape[0]
    hmask, qs, sc_raw = b[:, 0:32], b[:, 32:96], b[:, 96:108]
    d_all = _f16(b[:, 108:110].copy())
    aux = sc_raw.copy().view("<u4").astype(np.uint32)              # [n,3]
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
    a0, a1, tmp = aux[:, 0], aux[:, 1], aux[:, 2]
    n2 = ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4)
    n3 = ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)
    n0 = (a0 & k2) | (((tmp >> 0) & k1) << 4)
    n1 = (a1 & k2) | (((tmp >> 2) & k1) << 4)
    scales = np.stack([n0, n1, n2, n3], axis=1).astype("<u4").view(np.int8).reshape(n, 16).astype(np.float32)
    out = np.empty((n, 256), dtype=np.float32)
    is_, m = 0, 1
    for half in range(2):
        q = qs[:, 32 * half: 32 * half + 32]
        for j in range(4):
            shift = 2 * j
            for part in range(2):
                dl = d_all * (scales[:, is_:is_ + 1] - 32.0)
                ql = ((q[:, 16 * part: 16 * part + 16] >> shift) & 3).astype(np.int32)
                hm = (hmask[:, 16 * part: 16 * part + 16] & m) != 0
                v = (ql - np.where(hm, 0, 4)).astype(np.float32)
                y0 = 128 * half + j * 32 + 16 * part
                out[:, y0:y0 + 16] = dl * v
                is_ += 1
            m <<= 1
    return out


def _scale_min_k4(j, q):
    if j < 4:
        return (q[:, j] & 63), (q[:, j + 4] & 63)
    d = (q[:, j + 4] & 0xF) | ((q[:, j - 4] >> 6) << 4)
    m = (q[:, j + 4] >> 4) | ((q[:, j] >> 6) << 4)
    return d, m


def _dq_q4_k(b):
    n = b.shape[0]
    d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
    scales, qs = b[:, 4:16], b[:, 16:144]
    out = np.empty((n, 256), dtype=np.float32)
    for j in range(4):
        q = qs[:, 32 * j: 32 * j + 32]
        sc1, m1 = _scale_min_k4(2 * j, scales)
        sc2, m2 = _scale_min_k4(2 * j + 1, scales)
        d1, mm1 = d * sc1[:, None].astype(np.float32), dmin * m1[:, None].astype(np.float32)
        d2, mm2 = d * sc2[:, None].astype(np.float32), dmin * m2[:, None].astype(np.float32)
        out[:, 64 * j: 64 * j + 32] = d1 * (q & 0xF).astype(np.float32) - mm1
        out[:, 64 * j + 32: 64 * j + 64] = d2 * (q >> 4).astype(np.float32) - mm2
    return out


def _dq_q5_k(b):
    n = b.shape[0]
    d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
    scales, qh, qs = b[:, 4:16], b[:, 16:48], b[:, 48:176]
    out = np.empty((n, 256), dtype=np.float32)
    for j in range(4):
        ql = qs[:, 32 * j: 32 * j + 32]
        u1, u2 = 1 << (2 * j), 2 << (2 * j)
        sc1, m1 = _scale_min_k4(2 * j, scales)
        sc2, m2 = _scale_min_k4(2 * j + 1, scales)
        d1, mm1 = d * sc1[:, None].astype(np.float32), dmin * m1[:, None].astype(np.float32)
        d2, mm2 = d * sc2[:, None].astype(np.float32), dmin * m2[:, None].astype(np.float32)
        v1 = (ql & 0xF).astype(np.int32) + np.where((qh & u1) != 0, 16, 0)
        v2 = (ql >> 4).astype(np.int32) + np.where((qh & u2) != 0, 16, 0)
        out[:, 64 * j: 64 * j + 32] = d1 * v1.astype(np.float32) - mm1
        out[:, 64 * j + 32: 64 * j + 64] = d2 * v2.astype(np.float32) - mm2
    return out


def _dq_q6_k(b):
    n = b.shape[0]
    ql_all, qh_all = b[:, 0:128], b[:, 128:192]
    sc_all = b[:, 192:208].view(np.int8).astype(np.float32)
    d = _f16(b[:, 208:210].copy())
    out = np.empty((n, 256), dtype=np.float32)
    for half in range(2):
        ql, qh, sc = ql_all[:, 64 * half: 64 * half + 64], qh_all[:, 32 * half: 32 * half + 32], sc_all[:, 8 * half:]
        l = np.arange(32)
        is_ = l // 16
        q1 = ((ql[:, :32] & 0xF) | (((qh >> 0) & 3) << 4)).astype(np.int32) - 32
        q2 = ((ql[:, 32:64] & 0xF) | (((qh >> 2) & 3) << 4)).astype(np.int32) - 32
        q3 = ((ql[:, :32] >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int32) - 32
        q4 = ((ql[:, 32:64] >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int32) - 32
        y = 128 * half
        out[:, y + 0: y + 32] = d * sc[:, is_ + 0] * q1.astype(np.float32)
        out[:, y + 32: y + 64] = d * sc[:, is_ + 2] * q2.astype(np.float32)
        out[:, y + 64: y + 96] = d * sc[:, is_ + 4] * q3.astype(np.float32)
        out[:, y + 96: y + 128] = d * sc[:, is_ + 6] * q4.astype(np.float32)
    return out


def _dq_iq4_nl(b):
    d = _f16(b[:, 0:2].copy())
    qs = b[:, 2:18]
    return np.concatenate([KVALUES_IQ4NL[qs & 0xF], KVALUES_IQ4NL[qs >> 4]], axis=1) * d


def _dq_iq4_xs(b):
    n = b.shape[0]
    d = _f16(b[:, 0:2].copy())
    scales_h = b[:, 2:4].copy().view("<u2").astype(np.int32)      # [n,1]
    scales_l, qs = b[:, 4:8], b[:, 8:136]
    out = np.empty((n, 256), dtype=np.float32)
    for ib in range(8):
        ls = ((scales_l[:, ib // 2] >> (4 * (ib % 2))) & 0xF).astype(np.int32) | (((scales_h[:, 0] >> (2 * ib)) & 3) << 4)
        dl = d * (ls[:, None] - 32).astype(np.float32)
        q = qs[:, 16 * ib: 16 * ib + 16]
        out[:, 32 * ib: 32 * ib + 16] = dl * KVALUES_IQ4NL[q & 0xF]
        out[:, 32 * ib + 16: 32 * ib + 32] = dl * KVALUES_IQ4NL[q >> 4]
    return out


_DEQUANT = {"Q4_0": _dq_q4_0, "Q4_1": _dq_q4_1, "Q5_0": _dq_q5_0, "Q5_1": _dq_q5_1, "Q8_0": _dq_q8_0, "Q8_1": _dq_q8_1,
            "Q2_K": _dq_q2_k, "Q3_K": _dq_q3_k, "Q4_K": _dq_q4_k, "Q5_K": _dq_q5_k, "Q6_K": _dq_q6_k, "Q8_K": _dq_q8_k,
            "IQ4_NL": _dq_iq4_nl, "IQ4_XS": _dq_iq4_xs}
_PLAIN = {"F32": "<f4", "F64": "<f8", "I8": "i1", "I16": "<i2", "I32": "<i4", "I64": "<i8"}


def dequantize(raw: np.ndarray, type_name: str, count: int) -> np.ndarray:
    """Raw bytes of ``count`` values in ggml type ``type_name`` -> fp32 array of ``count`` values."""
    if type_name in _PLAIN:
        return raw.view(_PLAIN[type_name]).astype(np.float32)[:count]
    if type_name == "F16":
        return raw.view("<f2").astype(np.float32)[:count]
    if type_name == "BF16":
        return (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)[:count]
    fn = _DEQUANT.get(type_name)
    if fn is None:
        raise NotImplementedError(f"ggml type {type_name} is not de-quantised by this build "
                                  f"(supported: {sorted(list(_DEQUANT) + list(_PLAIN) + ['F16', 'BF16'])})")
    per, size = next((p, s) for (n, p, s) in TYPES.values() if n == type_name)
    blocks = raw.reshape(-1, size)
    return np.ascontiguousarray(fn(blocks), dtype=np.float32).reshape(-1)[:count]


# --------------------------------------------------------------------------- file
class GgufFile:
    def __init__(self, path: str):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        magic, version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        if version not in (2, 3):
            raise NotImplementedError(f"{path}: GGUF version {version} is not supported (2 and 3 are)")
        self.version = version
        n_tensors, n_kv = self._unpack("<QQ")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = self._string()
            (vt,) = self._unpack("<I")
            self.metadata[key] = self._value(vt)
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            ne = self._unpack("<" + "Q" * nd)
            tid, off = self._unpack("<IQ")
            if tid not in TYPES:
                raise NotImplementedError(f"{path}: tensor '{name}' has unknown ggml type {tid}")
            infos.append((name, tuple(reversed(ne)), tid, off))
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (self._pos + align - 1) // align * align
        self.tensors: Dict[str, GgufTensorInfo] = {
            name: GgufTensorInfo(name, shape, tid, self.data_start + off) for name, shape, tid, off in infos}

    # -- low-level reads
    def _unpack(self, fmt):
        size = struct.calcsize(fmt)
        vals = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += size
        return vals

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        s = self._mm[self._pos: self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, vt):
        simple = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
        if vt in simple:
            return self._unpack(simple[vt])[0]
        if vt == 8:
            return self._string()
        if vt == 9:
            et, n = self._unpack("<IQ")
            if et in simple and et != 7:
                fmt = simple[et]
                dt = np.dtype(fmt)
                arr = np.frombuffer(self._mm, dtype=dt, count=n, offset=self._pos).copy()
                self._pos += n * dt.itemsize
                return arr.tolist()
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {vt}")

    # -- tensors
    def raw(self, name: str) -> np.ndarray:
        info = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=info.nbytes, offset=info.offset)

    def read(self, name: str) -> torch.Tensor:
        """The tensor de-quantised to fp32, shaped outermost-first."""
        info = self.tensors[name]
        vals = dequantize(self.raw(name).copy(), info.type_name, info.count)
        return torch.from_numpy(vals.reshape(info.shape))

    def close(self):
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- model level
    @property
    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def decoder_spec(self):
        from ..models.spec import DecoderSpec, RopeSettings
        a, md = self.architecture, self.metadata

        def g(key, default=None):
            return md.get(f"{a}.{key}", default)

        dim = int(g("embedding_length"))
        heads = int(g("attention.head_count"))
        kv = g("attention.head_count_kv", heads)
        kv = int(kv[0] if isinstance(kv, list) else kv)
        head_dim = int(g("attention.key_length", dim // heads))
        vocab = int(g("vocab_size", len(md.get("tokenizer.ggml.tokens", [])) or 0))
        if vocab == 0 and "token_embd.weight" in self.tensors:
            vocab = self.tensors["token_embd.weight"].shape[0]
        rope = RopeSettings(theta=float(g("rope.freq_base", 10000.0)))
        if g("rope.dimension_count") and int(g("rope.dimension_count")) != head_dim:
            rope.rotary_dim = int(g("rope.dimension_count"))
        if g("rope.scaling.type") in ("linear", "yarn"):
            rope.scaling = g("rope.scaling.type")
            rope.factor = float(g("rope.scaling.factor", 1.0))
            rope.original_max_positions = g("rope.scaling.original_context_length")
        gemma = a.startswith("gemma")
        spec = DecoderSpec(
            vocabulary=vocab, dim=dim, layers=int(g("block_count")), heads=heads, kv_heads=kv, head_dim=head_dim,
            ff_dim=int(g("feed_forward_length")), max_positions=int(g("context_length", 2048)),
            norm="rms", norm_epsilon=float(g("attention.layer_norm_rms_epsilon", 1e-6)), gated=True,
            activation="gelu" if gemma else "silu", rope=rope,
            qkv_bias=any(n.endswith("attn_q.bias") for n in self.tensors),
            qk_norm=any(n.endswith("attn_q_norm.weight") for n in self.tensors),
            post_norms=any(n.endswith("post_attention_norm.weight") for n in self.tensors),
            tie_embeddings="output.weight" not in self.tensors,
            embedding_scale=float(dim) ** 0.5 if gemma else None,
            sliding_window=int(g("attention.sliding_window")) if g("attention.sliding_window") else None,
            attention_softcap=g("attn_logit_softcapping"), logit_softcap=g("final_logit_softcapping"),
            experts=int(g("expert_count", 0) or 0), experts_per_token=int(g("expert_used_count", 0) or 0))
        if gemma:
            spec.norm_offset = 0.0      # the converter stores Gemma's norm weights with the +1 already added
            if a == "gemma2":
                spec.sliding_window_layers = [i % 2 == 0 for i in range(spec.layers)]
            elif a == "gemma3":
                pattern = int(g("attention.sliding_window_pattern", 6))
                spec.sliding_window_layers = [(i + 1) % pattern != 0 for i in range(spec.layers)]
                if g("rope.freq_base_swa"):
                    spec.sliding_window_rope = RopeSettings(theta=float(g("rope.freq_base_swa")))
        return spec

    def idrak_tensors(self, spec=None) -> Dict[str, torch.Tensor]:
        """Tensors under the decoder's checkpoint names, ``[in, out]`` orientation."""
        spec = spec or self.decoder_spec()
        arch = self.architecture
        out: Dict[str, torch.Tensor] = {}

        def unpermute(w: torch.Tensor, n_head: int) -> torch.Tensor:
            # llama.cpp's converter interleaves the two halves of every head of q / k (its RoPE pairs neighbours);
            # undo it so the rotate-half convention of this package applies
            rows = w.shape[0]
            return (w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape))

        permuted = arch in ("llama", "mistral", "mixtral")
        simple = {"token_embd.weight": ("embed.weight", False), "output_norm.weight": ("norm.weight", False),
                  "output.weight": ("head.weight", True)}
        for src, (dst, tr) in simple.items():
            if src in self.tensors:
                t = self.read(src)
                out[dst] = t.t().contiguous() if tr else t
        per_layer = {"attn_norm.weight": ("attn_norm.weight", False), "ffn_norm.weight": ("mlp_norm.weight", False),
                     "attn_q.weight": ("attn.q.weight", True), "attn_k.weight": ("attn.k.weight", True),
                     "attn_v.weight": ("attn.v.weight", True), "attn_output.weight": ("attn.o.weight", True),
                     "attn_q.bias": ("attn.q.bias", False), "attn_k.bias": ("attn.k.bias", False),
                     "attn_v.bias": ("attn.v.bias", False), "attn_q_norm.weight": ("attn.q_norm.weight", False),
                     "attn_k_norm.weight": ("attn.k_norm.weight", False),
                     "ffn_gate.weight": ("mlp.gate.weight", True), "ffn_up.weight": ("mlp.up.weight", True),
                     "ffn_down.weight": ("mlp.down.weight", True),
                     "post_attention_norm.weight": ("post_attn_norm.weight", False),
                     "post_ffw_norm.weight": ("post_mlp_norm.weight", False)}
        for i in range(spec.layers):
            for src, (dst, tr) in per_layer.items():
                name = f"blk.{i}.{src}"
                if name not in self.tensors:
                    continue
                t = self.read(name)
                if permuted and src in ("attn_q.weight", "attn_q.bias"):
                    t = unpermute(t, spec.heads)
                if permuted and src in ("attn_k.weight", "attn_k.bias"):
                    t = unpermute(t, spec.kv_heads)
                out[f"layers.{i}.{dst}"] = t.t().contiguous() if tr else t
        if self.architecture.startswith("gemma"):
            # GGUF stores Gemma's norm weights with the +1 already added
            for k in list(out):
                if k.endswith("norm.weight"):
                    out[k] = out[k]
        return out
