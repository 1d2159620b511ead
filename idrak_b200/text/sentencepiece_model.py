"""SentencePiece ``.model`` files without the sentencepiece library: reader, writer, the precompiled character map
(a double-array trie over UTF-8 bytes plus a blob of replacement strings) and the bridge to this package's tokenizers.

A ``.model`` file is a protobuf ``ModelProto``: field 1 repeated pieces (piece, score, type), field 2 the trainer
settings (model kind, special ids, byte fallback), field 3 the normalizer settings (precompiled map, dummy prefix,
whitespace handling). ``read_model`` parses it with the package's own wire reader; ``to_tokenizer`` states it as the
equivalent ``tokenizer.json`` structure (Precompiled normalizer -> Metaspace pre-tokenizer -> Unigram / BPE model) and
returns the matching tokenizer class, so encoding goes through the same code as models that ship a ``tokenizer.json``.

Reference: SentencePieceReader.cs / SentencePieceWriter.cs, PrecompiledNormalizer.cs, DoubleArrayTrie.cs
(src/Idrak/Models/Tokenizers).
"""
from __future__ import annotations

import base64
import dataclasses
import struct
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from ..onnx.proto import Writer, fields

META = "▁"
TYPE_NORMAL, TYPE_UNKNOWN, TYPE_CONTROL, TYPE_USER, TYPE_UNUSED, TYPE_BYTE = 1, 2, 3, 4, 5, 6
MODEL_UNIGRAM, MODEL_BPE, MODEL_WORD, MODEL_CHAR = 1, 2, 3, 4


# --------------------------------------------------------------------------- double-array trie
class DoubleArrayTrie:
    """Double-array trie over byte strings in the unit layout SentencePiece's character maps use.

    One 32-bit unit per node: bits 0-7 label, bit 8 "a key ends below me", bit 9 "offset is stored in units of 256",
    bits 10-30 offset, bit 31 marks a value unit. The child of node ``n`` on byte ``c`` is ``n ^ offset(n) ^ c`` and is
    valid when its label is ``c``; the value of a key sits in the child reached with byte 0."""

    def __init__(self, units: Sequence[int]):
        self.units = list(units)

    @staticmethod
    def _offset(u: int) -> int:
        return (u >> 10) << ((u & (1 << 9)) >> 6)

    def common_prefixes(self, key: bytes, start: int = 0) -> List[Tuple[int, int]]:
        """Every key that is a prefix of ``key[start:]`` as (value, length), shortest first."""
        units, out = self.units, []
        pos = 0
        pos ^= self._offset(units[0])
        for i in range(start, len(key)):
            c = key[i]
            if c == 0:
                break
            pos ^= c
            if pos >= len(units):
                break
            u = units[pos]
            if (u & ((1 << 31) | 0xFF)) != c:
                break
            pos ^= self._offset(u)
            if (u >> 8) & 1:
                out.append((units[pos] & ((1 << 31) - 1), i + 1 - start))
        return out

    def lookup(self, key: bytes) -> Optional[int]:
        hits = [v for v, n in self.common_prefixes(key) if n == len(key)]
        return hits[0] if hits else None

    @classmethod
    def build(cls, entries: Dict[bytes, int]) -> "DoubleArrayTrie":
        """Builds the array for ``key -> value`` (keys without zero bytes, values below 2^31)."""
        keys = sorted(entries)
        if any(0 in k or not k for k in keys):
            raise ValueError("keys must be non-empty and free of zero bytes")
        units: List[int] = [0]
        used = [True]
        bases = set()

        def ensure(n):
            while len(units) <= n:
                units.append(0)
                used.append(False)

        # breadth-first over (node index, range of keys sharing the prefix, depth)
        work = [(0, 0, len(keys), 0)]
        while work:
            node, lo, hi, depth = work.pop()
            labels: List[Tuple[int, int, int]] = []          # (label, lo, hi); label 0 = a key ends here
            i = lo
            while i < hi:
                c = keys[i][depth] if depth < len(keys[i]) else 0
                j = i
                while j < hi and (keys[j][depth] if depth < len(keys[j]) else 0) == c:
                    j += 1
                labels.append((c, i, j))
                i = j
            # first base no other node uses (a slot is recognised by its label alone, so two nodes sharing a base
            # would see each other's children) whose child slots are all free
            base = 1
            while True:
                if base not in bases and all((base ^ c) >= len(used) or not used[base ^ c] for c, _, _ in labels) and \
                        all((base ^ c) != 0 for c, _, _ in labels):
                    break
                base += 1
            bases.add(base)
            rel = node ^ base
            if rel >= 1 << 21:
                raise ValueError("trie too large for the plain offset form")
            units[node] |= rel << 10
            for c, a, b in labels:
                child = base ^ c
                ensure(child)
                used[child] = True
                if c == 0:
                    units[node] |= 1 << 8
                    units[child] = (1 << 31) | entries[keys[a]]
                else:
                    units[child] = c
                    work.append((child, a, b, depth + 1))
        return cls(units)

    def to_bytes(self) -> bytes:
        return struct.pack(f"<{len(self.units)}I", *self.units)


# --------------------------------------------------------------------------- precompiled normalizer
class PrecompiledNormalizer:
    """``precompiled_charsmap``: u32 trie size in bytes, the trie units, then a blob of zero-terminated replacement
    strings. Normalization walks the text: at each position the longest key of the trie is replaced by its string;
    where no key matches, one character is copied."""

    def __init__(self, charsmap: bytes):
        self.raw = bytes(charsmap)
        if len(self.raw) < 4:
            self.trie, self.blob = None, b""
            return
        (size,) = struct.unpack_from("<I", self.raw, 0)
        if size % 4 or 4 + size > len(self.raw):
            raise ValueError("precompiled character map: trie size does not fit the data")
        self.trie = DoubleArrayTrie(struct.unpack_from(f"<{size // 4}I", self.raw, 4))
        self.blob = self.raw[4 + size:]

    @classmethod
    def from_rules(cls, rules: Dict[str, str]) -> "PrecompiledNormalizer":
        blob, entries = bytearray(), {}
        for src, dst in sorted(rules.items()):
            entries[src.encode("utf-8")] = len(blob)
            blob += dst.encode("utf-8") + b"\0"
        trie = DoubleArrayTrie.build(entries).to_bytes() if entries else b""
        return cls(struct.pack("<I", len(trie)) + trie + bytes(blob))

    def _replacement(self, at: int) -> bytes:
        end = self.blob.index(b"\0", at)
        return self.blob[at:end]

    def __call__(self, text: str) -> str:
        if self.trie is None:
            return text
        data, out, i = text.encode("utf-8"), bytearray(), 0
        while i < len(data):
            hits = self.trie.common_prefixes(data, i)
            if hits:
                value, n = hits[-1]
                out += self._replacement(value)
                i += n
                continue
            n = 1
            while i + n < len(data) and (data[i + n] & 0xC0) == 0x80:
                n += 1
            out += data[i:i + n]
            i += n
        return out.decode("utf-8", errors="replace")


# --------------------------------------------------------------------------- the model file
@dataclasses.dataclass
class SentencePieceModel:
    pieces: List[str]
    scores: List[float]
    types: List[int]
    model_type: int = MODEL_UNIGRAM
    unk_id: int = 0
    bos_id: int = 1
    eos_id: int = 2
    pad_id: int = -1
    byte_fallback: bool = False
    normalizer_name: str = ""
    precompiled_charsmap: bytes = b""
    add_dummy_prefix: bool = True
    remove_extra_whitespaces: bool = True
    escape_whitespaces: bool = True
    treat_whitespace_as_suffix: bool = False

    @property
    def vocab_size(self) -> int:
        return len(self.pieces)


def _bool(v, default):
    return default if v is None else bool(v)


def read_model(path_or_bytes) -> SentencePieceModel:
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    pieces, scores, types = [], [], []
    trainer: Dict[int, object] = {}
    norm: Dict[int, object] = {}
    for num, wire, v in fields(bytes(data)):
        if num == 1 and wire == 2:
            piece, score, kind = "", 0.0, TYPE_NORMAL
            for n2, w2, v2 in fields(v):
                if n2 == 1:
                    piece = v2.decode("utf-8")
                elif n2 == 2:
                    score = struct.unpack("<f", struct.pack("<I", v2))[0] if isinstance(v2, int) else struct.unpack("<f", v2)[0]
                elif n2 == 3:
                    kind = int(v2)
            pieces.append(piece)
            scores.append(score)
            types.append(kind)
        elif num == 2 and wire == 2:
            for n2, w2, v2 in fields(v):
                trainer[n2] = v2
        elif num == 3 and wire == 2:
            for n2, w2, v2 in fields(v):
                norm[n2] = v2
    if not pieces:
        raise ValueError("sentencepiece model: no pieces (not a ModelProto?)")

    def signed(v, default):
        if v is None:
            return default
        v = int(v)
        return v - (1 << 64) if v >= 1 << 63 else v
    return SentencePieceModel(
        pieces, scores, types, int(trainer.get(3, MODEL_UNIGRAM)), signed(trainer.get(40), 0), signed(trainer.get(41), 1),
        signed(trainer.get(42), 2), signed(trainer.get(43), -1), _bool(trainer.get(35), False),
        norm.get(1, b"").decode("utf-8") if isinstance(norm.get(1, b""), bytes) else "", bytes(norm.get(2, b"")),
        _bool(norm.get(3), True), _bool(norm.get(4), True), _bool(norm.get(5), True), _bool(trainer.get(24), False))


def write_model(model: SentencePieceModel, path: Optional[str] = None) -> bytes:
    w = Writer()
    for piece, score, kind in zip(model.pieces, model.scores, model.types):
        p = Writer()
        p.string(1, piece)
        p.float32(2, score)
        if kind != TYPE_NORMAL:
            p.varint(3, kind)
        w.bytes(1, p.done())
    t = Writer()
    t.varint(3, model.model_type)
    t.varint(4, len(model.pieces))
    if model.treat_whitespace_as_suffix:
        t.varint(24, 1)
    if model.byte_fallback:
        t.varint(35, 1)
    for num, v in ((40, model.unk_id), (41, model.bos_id), (42, model.eos_id), (43, model.pad_id)):
        t.varint(num, v & ((1 << 64) - 1))
    w.bytes(2, t.done())
    n = Writer()
    if model.normalizer_name:
        n.string(1, model.normalizer_name)
    if model.precompiled_charsmap:
        n.bytes(2, model.precompiled_charsmap)
    n.varint(3, int(model.add_dummy_prefix))
    n.varint(4, int(model.remove_extra_whitespaces))
    n.varint(5, int(model.escape_whitespaces))
    w.bytes(3, n.done())
    out = w.done()
    if path is not None:
        with open(path, "wb") as f:
            f.write(out)
    return out


def tokenizer_spec(model: SentencePieceModel) -> dict:
    """The ``tokenizer.json`` structure that encodes like this model."""
    normalizers = []
    if model.precompiled_charsmap:
        normalizers.append({"type": "Precompiled",
                            "precompiled_charsmap": base64.b64encode(model.precompiled_charsmap).decode("ascii")})
    if model.remove_extra_whitespaces:
        normalizers.append({"type": "Strip", "strip_left": True, "strip_right": True})
        normalizers.append({"type": "Replace", "pattern": {"Regex": " {2,}"}, "content": " "})
    added = [{"id": i, "content": p, "special": True} for i, (p, k) in enumerate(zip(model.pieces, model.types))
             if k in (TYPE_CONTROL, TYPE_UNKNOWN)]
    added += [{"id": i, "content": p, "special": False} for i, (p, k) in enumerate(zip(model.pieces, model.types))
              if k == TYPE_USER]
    spec = {
        "normalizer": {"type": "Sequence", "normalizers": normalizers} if normalizers else None,
        "pre_tokenizer": {"type": "Metaspace", "replacement": META,
                          "prepend_scheme": "always" if model.add_dummy_prefix else "never", "split": True},
        "decoder": {"type": "Metaspace", "replacement": META},
        "added_tokens": added,
    }
    if model.model_type == MODEL_UNIGRAM:
        spec["model"] = {"type": "Unigram", "unk_id": model.unk_id if model.unk_id >= 0 else None,
                         "vocab": [[p, s] for p, s in zip(model.pieces, model.scores)],
                         "byte_fallback": model.byte_fallback}
    elif model.model_type == MODEL_BPE:
        vocab = {p: i for i, p in enumerate(model.pieces)}
        # a BPE piece was made by its best-scoring split into two existing pieces; merges in order of piece score
        merges = []
        order = sorted((i for i, k in enumerate(model.types) if k == TYPE_NORMAL and len(model.pieces[i]) > 1),
                       key=lambda i: -model.scores[i])
        rank = {model.pieces[i]: r for r, i in enumerate(order)}
        for i in order:
            p, best = model.pieces[i], None
            for cut in range(1, len(p)):
                a, b = p[:cut], p[cut:]
                if a in vocab and b in vocab:
                    cost = max(rank.get(a, -1), rank.get(b, -1))
                    if cost < rank[p] and (best is None or cost < best[0]):
                        best = (cost, a, b)
            if best is not None:
                merges.append(f"{best[1]} {best[2]}")
        spec["model"] = {"type": "BPE", "vocab": vocab, "merges": merges, "byte_fallback": model.byte_fallback,
                         "unk_token": model.pieces[model.unk_id] if 0 <= model.unk_id < len(model.pieces) else None}
    else:
        raise ValueError(f"sentencepiece model kind {model.model_type} (word / char) has no tokenizer here")
    return spec


def to_tokenizer(model: SentencePieceModel):
    from .tokenizers_native import BpeTokenizer, UnigramTokenizer
    spec = tokenizer_spec(model)
    config = {}
    for name, i in (("bos_token", model.bos_id), ("eos_token", model.eos_id), ("pad_token", model.pad_id)):
        if 0 <= i < len(model.pieces):
            config[name] = model.pieces[i]
    cls = UnigramTokenizer if model.model_type == MODEL_UNIGRAM else BpeTokenizer
    return cls(spec, config)


def load_sentencepiece(path: str):
    """Tokenizer from a ``.model`` file."""
    return to_tokenizer(read_model(path))


def from_unigram(pieces: Iterable[Tuple[str, float]], specials: Sequence[str] = ("<unk>", "<s>", "</s>"),
                 byte_fallback: bool = False, rules: Optional[Dict[str, str]] = None) -> SentencePieceModel:
    """A model from trained (piece, score) pairs: specials first (unknown, begin, end), then byte pieces, then pieces."""
    names, scores, types = list(specials), [0.0] * len(specials), [TYPE_UNKNOWN] + [TYPE_CONTROL] * (len(specials) - 1)
    if byte_fallback:
        for b in range(256):
            names.append(f"<0x{b:02X}>")
            scores.append(0.0)
            types.append(TYPE_BYTE)
    for p, s in pieces:
        if p in specials:
            continue
        names.append(p)
        scores.append(float(s))
        types.append(TYPE_NORMAL)
    charsmap = PrecompiledNormalizer.from_rules(rules).raw if rules else b""
    return SentencePieceModel(names, scores, types, MODEL_UNIGRAM, 0, 1 if len(specials) > 1 else -1,
                              2 if len(specials) > 2 else -1, -1, byte_fallback, "user" if rules else "identity", charsmap)
