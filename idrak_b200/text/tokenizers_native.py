"""This package's own tokenizer runtimes: byte-pair encoding (merge loop in the native library, `csrc/bpe.cpp`),
WordPiece (greedy longest match) and Unigram (Viterbi over piece scores), read from the ``tokenizer.json`` layout, plus
a BPE trainer that writes the same layout.

    tok = load_tokenizer_json("tokenizer.json")        # BpeTokenizer / WordPieceTokenizer / UnigramTokenizer
    ids = tok.encode("Hello world")
    text = tok.decode(ids)
    tok = train_bpe(lines, vocab_size=4096, special_tokens=["<|endoftext|>"]); tok.save("tokenizer.json")

Supported pieces of the layout: normalizers NFC / NFD / NFKC / NFKD / Lowercase / Strip / StripAccents / Replace /
Prepend / BertNormalizer / Sequence; pre-tokenizers ByteLevel / Split / Whitespace / WhitespaceSplit / Metaspace /
BertPreTokenizer / Digits / Punctuation / Sequence; byte fallback; added and special tokens. Anything else is refused by name.

Reference: src/Idrak/Models/BpeTokenizer.cs (byte-level and SentencePiece-style BPE from tokenizer.json or GGUF),
src/Idrak/Models/BpeTrainer.cs, Tokenizers/UnigramTokenizer.cs, Tokenizers/WordPieceTokenizer.cs and the
normalizer / pre-tokenizer registries beside them.
"""
from __future__ import annotations

import ctypes as C
import json
import unicodedata
from collections import Counter, defaultdict
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import regex

from .tokenizer import Tokenizer

GPT2_PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
META = "▁"


def bytes_to_unicode() -> Dict[int, str]:
    """The printable stand-in for each byte used by byte-level vocabularies."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


BYTE_CHAR = bytes_to_unicode()
CHAR_BYTE = {c: b for b, c in BYTE_CHAR.items()}


# --------------------------------------------------------------------------------------------- normalizers
def _strip_accents(s: str) -> str:
    return "".join(c for c in unicodedata.normalize("NFD", s) if unicodedata.category(c) != "Mn")


def _is_cjk(cp: int) -> bool:
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0x2A700 <= cp <= 0x2B73F
            or 0x2B740 <= cp <= 0x2B81F or 0x2B820 <= cp <= 0x2CEAF or 0xF900 <= cp <= 0xFAFF or 0x2F800 <= cp <= 0x2FA1F)


def _bert_normalizer(d: dict) -> Callable[[str], str]:
    clean, chinese, lower = d.get("clean_text", True), d.get("handle_chinese_chars", True), d.get("lowercase", True)
    strip = d.get("strip_accents")
    strip = lower if strip is None else strip

    def run(s: str) -> str:
        if clean:
            s = "".join(" " if c.isspace() else c for c in s
                        if not (ord(c) == 0 or ord(c) == 0xFFFD or (unicodedata.category(c).startswith("C") and c not in "\t\n\r")))
        if chinese:
            s = "".join(f" {c} " if _is_cjk(ord(c)) else c for c in s)
        if strip:
            s = _strip_accents(s)
        if lower:
            s = s.lower()
        return s
    return run


def _pattern(p) -> "regex.Pattern":
    if isinstance(p, dict):
        return regex.compile(p["Regex"]) if "Regex" in p else regex.compile(regex.escape(p["String"]))
    return regex.compile(regex.escape(p))


def build_normalizer(d: Optional[dict]) -> Callable[[str], str]:
    if not d:
        return lambda s: s
    t = d["type"]
    if t == "Sequence":
        parts = [build_normalizer(x) for x in d["normalizers"]]

        def seq(s):
            for p in parts:
                s = p(s)
            return s
        return seq
    if t in ("NFC", "NFD", "NFKC", "NFKD"):
        return lambda s: unicodedata.normalize(t, s)
    if t == "Lowercase":
        return str.lower
    if t == "Strip":
        left, right = d.get("strip_left", True), d.get("strip_right", True)
        return lambda s: (s.lstrip() if left else s).rstrip() if right else (s.lstrip() if left else s)
    if t == "StripAccents":
        return _strip_accents
    if t == "Replace":
        pat, content = _pattern(d["pattern"]), d["content"]
        return lambda s: pat.sub(lambda m: content, s)
    if t == "Prepend":
        pre = d["prepend"]
        return lambda s: pre + s if s else s
    if t == "BertNormalizer":
        return _bert_normalizer(d)
    if t == "Precompiled":
        # SentencePiece's compiled character map (T5, ALBERT, XLM-R ...): base64 of [trie | replacement strings]
        import base64
        from .sentencepiece_model import PrecompiledNormalizer
        return PrecompiledNormalizer(base64.b64decode(d["precompiled_charsmap"]))
    raise ValueError(f"tokenizer.json: normalizer {t!r} is not supported")


# --------------------------------------------------------------------------------------------- pre-tokenizers
def _is_punct(c: str) -> bool:
    cp = ord(c)
    return (33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126) or unicodedata.category(c).startswith("P")


def _split_isolated(pat, words: List[str], invert: bool = False, behavior: str = "Isolated") -> List[str]:
    out = []
    for w in words:
        pos = 0
        pieces: List[Tuple[str, bool]] = []           # (text, is a match)
        for m in pat.finditer(w):
            if m.end() == m.start():
                continue
            if m.start() > pos:
                pieces.append((w[pos:m.start()], False))
            pieces.append((m.group(), True))
            pos = m.end()
        if pos < len(w):
            pieces.append((w[pos:], False))
        if invert:
            pieces = [(t, not f) for t, f in pieces]
        if behavior == "Removed":
            out += [t for t, f in pieces if not f]
        elif behavior == "MergedWithPrevious":
            cur = ""
            for t, f in pieces:
                cur += t
                if f:
                    out.append(cur)
                    cur = ""
            if cur:
                out.append(cur)
        elif behavior == "MergedWithNext":
            cur = ""
            for t, f in pieces:
                if f:
                    cur += t
                else:
                    out.append(cur + t)
                    cur = ""
            if cur:
                out.append(cur)
        else:                                           # Isolated (and Contiguous for single matches)
            out += [t for t, _ in pieces]
    return [x for x in out if x]


def build_pre_tokenizer(d: Optional[dict]) -> Tuple[Callable[[List[str]], List[str]], bool]:
    """Returns (function from a list of strings to a list of pre-tokens, whether the words end up byte-level mapped)."""
    if not d:
        return (lambda ws: ws), False
    t = d["type"]
    if t == "Sequence":
        parts = [build_pre_tokenizer(x) for x in d["pretokenizers"]]

        def seq(ws):
            for f, _ in parts:
                ws = f(ws)
            return ws
        return seq, any(b for _, b in parts)
    if t == "ByteLevel":
        pat = regex.compile(GPT2_PATTERN) if d.get("use_regex", True) else None
        prefix = d.get("add_prefix_space", False)

        def byte_level(ws):
            if prefix and ws and ws[0] and not ws[0].startswith(" "):
                ws = [" " + ws[0]] + ws[1:]
            if pat is not None:
                ws = [m for w in ws for m in pat.findall(w)]
            return ["".join(BYTE_CHAR[b] for b in w.encode("utf-8")) for w in ws]
        return byte_level, True
    if t == "Split":
        pat = _pattern(d["pattern"])
        return (lambda ws: _split_isolated(pat, ws, d.get("invert", False), d.get("behavior", "Isolated"))), False
    if t == "Whitespace":
        pat = regex.compile(r"\w+|[^\w\s]+")
        return (lambda ws: [m for w in ws for m in pat.findall(w)]), False
    if t == "WhitespaceSplit":
        return (lambda ws: [m for w in ws for m in w.split()]), False
    if t == "Metaspace":
        rep = d.get("replacement", META)
        scheme = d.get("prepend_scheme", "always" if d.get("add_prefix_space", True) else "never")
        split = d.get("split", True)

        def metaspace(ws):
            out = []
            for i, w in enumerate(ws):
                w = w.replace(" ", rep)
                if w and not w.startswith(rep) and (scheme == "always" or (scheme == "first" and i == 0)):
                    w = rep + w
                if split:
                    out += [m for m in regex.findall(f"{regex.escape(rep)}?[^{regex.escape(rep)}]*", w) if m]
                else:
                    out.append(w)
            return out
        return metaspace, False
    if t == "BertPreTokenizer":
        def bert(ws):
            out = []
            for w in ws:
                for part in w.split():
                    cur = ""
                    for c in part:
                        if _is_punct(c):
                            if cur:
                                out.append(cur)
                                cur = ""
                            out.append(c)
                        else:
                            cur += c
                    if cur:
                        out.append(cur)
            return out
        return bert, False
    if t == "Digits":
        pat = regex.compile(r"\p{Nd}" if d.get("individual_digits", False) else r"\p{Nd}+")
        return (lambda ws: _split_isolated(pat, ws)), False
    if t == "Punctuation":
        pat = regex.compile(r"\p{P}|[\x21-\x2F\x3A-\x40\x5B-\x60\x7B-\x7E]")
        return (lambda ws: _split_isolated(pat, ws, behavior=d.get("behavior", "Isolated"))), False
    raise ValueError(f"tokenizer.json: pre-tokenizer {t!r} is not supported")


# --------------------------------------------------------------------------------------------- shared base
class JsonTokenizer(Tokenizer):
    """What the three model kinds share: added tokens, normalizer, pre-tokenizer, decoding and special-token facts."""

    def __init__(self, spec: dict, config: Optional[dict] = None):
        self.spec = spec
        model = spec["model"]
        self.normalize = build_normalizer(spec.get("normalizer"))
        self.pre_tokenize, self.byte_level = build_pre_tokenizer(spec.get("pre_tokenizer"))
        self.added = {a["content"]: int(a["id"]) for a in spec.get("added_tokens", [])}
        self.special_tokens = {a["content"]: int(a["id"]) for a in spec.get("added_tokens", []) if a.get("special")}
        self._added_pat = (regex.compile("|".join(regex.escape(k) for k in sorted(self.added, key=len, reverse=True)))
                           if self.added else None)
        self.byte_fallback = bool(model.get("byte_fallback", False))
        dec = spec.get("decoder") or {}
        kinds = [dec.get("type")] + [x.get("type") for x in dec.get("decoders", [])] if dec else []
        self._decode_kind = ("bytelevel" if "ByteLevel" in kinds or self.byte_level else
                             "wordpiece" if "WordPiece" in kinds else
                             "metaspace" if ("Metaspace" in kinds or "ByteFallback" in kinds or self.byte_fallback
                                             or (spec.get("pre_tokenizer") or {}).get("type") == "Metaspace") else "plain")
        self._fill_vocab(model)
        self.id_to_token = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.added.items()})
        config = config or {}
        self.chat_template = config.get("chat_template") if isinstance(config.get("chat_template"), str) else None

        def tid(name):
            v = config.get(name)
            v = v.get("content") if isinstance(v, dict) else v
            return self.token_to_id(v) if isinstance(v, str) else None
        self.bos_token_id, self.pad_token_id = tid("bos_token"), tid("pad_token")
        eos = tid("eos_token")
        self.eos_token_ids = (eos,) if eos is not None else ()

    # subclasses: set self.vocab and whatever the model needs; encode one pre-token
    def _fill_vocab(self, model: dict) -> None:
        raise NotImplementedError

    def _encode_words(self, words: List[str]) -> List[int]:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        return max(self.id_to_token) + 1 if self.id_to_token else 0

    def token_to_id(self, token: str) -> Optional[int]:
        return self.added.get(token, self.vocab.get(token))

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids: List[int] = []
        pos = 0
        spans: List[Tuple[str, Optional[int]]] = []
        if self._added_pat is not None:
            for m in self._added_pat.finditer(text):
                if m.start() > pos:
                    spans.append((text[pos:m.start()], None))
                spans.append((m.group(), self.added[m.group()]))
                pos = m.end()
        if pos < len(text):
            spans.append((text[pos:], None))
        for piece, tid in spans:
            if tid is not None:
                ids.append(tid)
                continue
            piece = self.normalize(piece)
            if piece:
                ids += self._encode_words(self.pre_tokenize([piece]))
        if add_special_tokens and self.bos_token_id is not None:
            ids = [self.bos_token_id] + ids
        return ids

    def _byte_fallback_ids(self, ch: str) -> Optional[List[int]]:
        out = []
        for b in ch.encode("utf-8"):
            i = self.vocab.get(f"<0x{b:02X}>")
            if i is None:
                return None
            out.append(i)
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        special = set(self.special_tokens.values())
        toks = [self.id_to_token.get(int(i), "") for i in ids if not (skip_special_tokens and int(i) in special)]
        if self._decode_kind == "bytelevel":
            buf = bytearray()
            for t in toks:
                if all(c in CHAR_BYTE for c in t):
                    buf += bytes(CHAR_BYTE[c] for c in t)
                else:
                    buf += t.encode("utf-8")            # an added token written in plain characters
            return buf.decode("utf-8", errors="replace")
        if self._decode_kind == "wordpiece":
            prefix = self.spec["model"].get("continuing_subword_prefix", "##")
            out = ""
            for t in toks:
                out += t[len(prefix):] if t.startswith(prefix) and out else (" " + t if out else t)
            for a, b in ((" .", "."), (" ?", "?"), (" !", "!"), (" ,", ","), (" ' ", "'"), (" n't", "n't"), (" 'm", "'m"),
                         (" 's", "'s"), (" 've", "'ve"), (" 're", "'re")):
                out = out.replace(a, b)
            return out
        if self._decode_kind == "metaspace":
            buf = bytearray()
            for t in toks:
                if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                    buf.append(int(t[3:5], 16))
                else:
                    buf += t.replace(META, " ").encode("utf-8")
            s = buf.decode("utf-8", errors="replace")
            return s[1:] if s.startswith(" ") else s
        return "".join(toks)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.spec, f, ensure_ascii=False)


# --------------------------------------------------------------------------------------------- BPE
class BpeTokenizer(JsonTokenizer):
    """Byte-pair encoding; the merge loop runs in the native library when it is built, else in Python."""

    def _fill_vocab(self, model: dict) -> None:
        self.vocab: Dict[str, int] = {k: int(v) for k, v in model["vocab"].items()}
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
        self.unk_id = self.vocab.get(model.get("unk_token")) if model.get("unk_token") else None
        self.ignore_merges = bool(model.get("ignore_merges", False))
        self.suffix = model.get("end_of_word_suffix") or ""
        left, right, merged = [], [], []
        for a, b in merges:
            ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
            if ia is None or ib is None or im is None:   # a rule whose pieces are not in the vocabulary can never apply
                ia, ib, im = -1, -1, -1
            left.append(ia), right.append(ib), merged.append(im)
        self._rules = {(a, b): (r, m) for r, (a, b, m) in reversed(list(enumerate(zip(left, right, merged)))) if a >= 0}
        self._handle = None
        self._lib = None
        try:
            from .. import _native
            if _native.available():
                i32p, i64p = C.POINTER(C.c_int32), C.POINTER(C.c_int64)
                self._create = _native.bind("idrak_bpe_create", C.c_void_p, [i32p, i32p, i32p, C.c_int64])
                self._free = _native.bind("idrak_bpe_free", None, [C.c_void_p])
                self._encode = _native.bind("idrak_bpe_encode", C.c_int64, [C.c_void_p, i32p, i64p, C.c_int64, i32p, i64p])
                arrs = [np.asarray(x, dtype=np.int32) for x in (left, right, merged)]
                self._handle = self._create(*[a.ctypes.data_as(i32p) for a in arrs], len(left))
                self._lib = True
        except (OSError, AttributeError):
            self._handle = None

    def __del__(self):
        if getattr(self, "_handle", None):
            try:
                self._free(self._handle)
            except Exception:
                pass
            self._handle = None

    @property
    def native(self) -> bool:
        return self._handle is not None

    def _symbols(self, word: str) -> List[int]:
        out = []
        chars = list(word)
        for i, ch in enumerate(chars):
            t = ch + self.suffix if self.suffix and i == len(chars) - 1 else ch
            tid = self.vocab.get(t)
            if tid is None:
                fb = self._byte_fallback_ids(ch) if self.byte_fallback else None
                if fb is not None:
                    out += fb
                elif self.unk_id is not None:
                    if not out or out[-1] != self.unk_id:       # runs of unknown characters fuse into one
                        out.append(self.unk_id)
            else:
                out.append(tid)
        return out

    def _merge_python(self, w: List[int]) -> List[int]:
        while len(w) > 1:
            best = min(((self._rules.get((w[i], w[i + 1]), (1 << 30, 0))[0], i) for i in range(len(w) - 1)))
            if best[0] == 1 << 30:
                break
            a, b = w[best[1]], w[best[1] + 1]
            m = self._rules[(a, b)][1]
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(m)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            w = out
        return w

    def _encode_words(self, words: List[str]) -> List[int]:
        whole: Dict[int, int] = {}
        syms: List[List[int]] = []
        for k, w in enumerate(words):
            if self.ignore_merges and w in self.vocab:
                whole[k] = self.vocab[w]
                syms.append([])
            else:
                syms.append(self._symbols(w))
        if self._handle is None:
            merged = [self._merge_python(list(s)) if s else [] for s in syms]
        else:
            flat = np.fromiter((x for s in syms for x in s), dtype=np.int32, count=sum(len(s) for s in syms))
            offs = np.zeros(len(syms) + 1, dtype=np.int64)
            np.cumsum([len(s) for s in syms], out=offs[1:])
            out = np.empty(max(len(flat), 1), dtype=np.int32)
            out_offs = np.empty(len(syms) + 1, dtype=np.int64)
            i32p, i64p = C.POINTER(C.c_int32), C.POINTER(C.c_int64)
            self._encode(self._handle, flat.ctypes.data_as(i32p), offs.ctypes.data_as(i64p), len(syms),
                         out.ctypes.data_as(i32p), out_offs.ctypes.data_as(i64p))
            merged = [out[out_offs[k]:out_offs[k + 1]].tolist() for k in range(len(syms))]
        ids: List[int] = []
        for k, m in enumerate(merged):
            if k in whole:
                ids.append(whole[k])
            else:
                ids += m
        return ids


# --------------------------------------------------------------------------------------------- WordPiece
class WordPieceTokenizer(JsonTokenizer):
    def _fill_vocab(self, model: dict) -> None:
        self.vocab = {k: int(v) for k, v in model["vocab"].items()}
        self.prefix = model.get("continuing_subword_prefix", "##")
        self.unk_id = self.vocab[model.get("unk_token", "[UNK]")]
        self.max_chars = int(model.get("max_input_chars_per_word", 100))

    def _encode_words(self, words: List[str]) -> List[int]:
        ids: List[int] = []
        for w in words:
            if len(w) > self.max_chars:
                ids.append(self.unk_id)
                continue
            start, piece_ids = 0, []
            while start < len(w):
                end, found = len(w), None
                while end > start:
                    sub = w[start:end] if start == 0 else self.prefix + w[start:end]
                    found = self.vocab.get(sub)
                    if found is not None:
                        break
                    end -= 1
                if found is None:
                    piece_ids = [self.unk_id]
                    break
                piece_ids.append(found)
                start = end
            ids += piece_ids
        return ids


# --------------------------------------------------------------------------------------------- Unigram
class UnigramTokenizer(JsonTokenizer):
    def _fill_vocab(self, model: dict) -> None:
        pieces = model["vocab"]
        self.vocab = {p: i for i, (p, _) in enumerate(pieces)}
        self.scores = [float(s) for _, s in pieces]
        self.unk_id = model.get("unk_id")
        self.max_len = max((len(p) for p, _ in pieces), default=1)
        low = min(self.scores) if self.scores else 0.0
        self.unk_score = low - 10.0

    def _encode_words(self, words: List[str]) -> List[int]:
        ids: List[int] = []
        for w in words:
            n = len(w)
            best = [float("-inf")] * (n + 1)
            back: List[Tuple[int, Optional[int]]] = [(0, None)] * (n + 1)
            best[0] = 0.0
            for i in range(n):
                if best[i] == float("-inf"):
                    continue
                single = False
                for j in range(i + 1, min(n, i + self.max_len) + 1):
                    tid = self.vocab.get(w[i:j])
                    if tid is None:
                        continue
                    if j == i + 1:
                        single = True
                    s = best[i] + self.scores[tid]
                    if s > best[j]:
                        best[j], back[j] = s, (i, tid)
                if not single:                                   # no piece covers this character alone: unknown
                    s = best[i] + self.unk_score
                    if s > best[i + 1]:
                        best[i + 1], back[i + 1] = s, (i, -1)
            out: List[int] = []
            j = n
            while j > 0:
                i, tid = back[j]
                if tid == -1:
                    fb = self._byte_fallback_ids(w[i:j]) if self.byte_fallback else None
                    if fb is not None:
                        out += reversed(fb)
                    elif self.unk_id is not None and not (out and out[-1] == self.unk_id):
                        out.append(self.unk_id)                  # adjacent unknowns fuse
                else:
                    out.append(tid)
                j = i
            ids += reversed(out)
        return ids


def load_tokenizer_json(path: str, config: Optional[dict] = None) -> JsonTokenizer:
    with open(path, "r", encoding="utf-8") as f:
        spec = json.load(f)
    kind = spec["model"].get("type") or ("Unigram" if isinstance(spec["model"].get("vocab"), list) else
                                         "BPE" if "merges" in spec["model"] else "WordPiece")
    cls = {"BPE": BpeTokenizer, "WordPiece": WordPieceTokenizer, "Unigram": UnigramTokenizer}.get(kind)
    if cls is None:
        raise ValueError(f"tokenizer.json: model type {kind!r} is not supported")
    return cls(spec, config)


# --------------------------------------------------------------------------------------------- BPE trainer
def train_bpe(texts: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = (), min_frequency: int = 2,
              pattern: str = GPT2_PATTERN) -> BpeTokenizer:
    """Byte-level BPE: count pre-tokens, then repeatedly merge the most frequent adjacent pair (ties: the smaller pair
    in the order of its strings), updating only the words that contain it."""
    pat = regex.compile(pattern)
    counts: Counter = Counter()
    for t in texts:
        for m in pat.findall(t):
            counts["".join(BYTE_CHAR[b] for b in m.encode("utf-8"))] += 1
    vocab: Dict[str, int] = {}
    for s in special_tokens:
        vocab.setdefault(s, len(vocab))
    first = len(vocab)
    for b in range(256):
        vocab.setdefault(BYTE_CHAR[b], len(vocab))
    words = [list(w) for w in counts]
    freqs = [counts[w] for w in counts]
    pairs: Counter = Counter()
    where: Dict[Tuple[str, str], set] = defaultdict(set)
    for k, (w, f) in enumerate(zip(words, freqs)):
        for a, b in zip(w, w[1:]):
            pairs[(a, b)] += f
            where[(a, b)].add(k)
    merges: List[Tuple[str, str]] = []
    while len(vocab) < vocab_size and pairs:
        top = max(pairs.values())
        if top < min_frequency:
            break
        a, b = min(p for p, c in pairs.items() if c == top)
        merges.append((a, b))
        vocab.setdefault(a + b, len(vocab))
        for k in list(where.pop((a, b), ())):
            w, f = words[k], freqs[k]
            for x, y in zip(w, w[1:]):
                pairs[(x, y)] -= f
                if pairs[(x, y)] <= 0:
                    del pairs[(x, y)]
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            words[k] = out
            for x, y in zip(out, out[1:]):
                pairs[(x, y)] += f
                where[(x, y)].add(k)
        pairs.pop((a, b), None)
    spec = {
        "version": "1.0", "truncation": None, "padding": None,
        "added_tokens": [{"id": vocab[s], "content": s, "single_word": False, "lstrip": False, "rstrip": False,
                          "normalized": False, "special": True} for s in special_tokens],
        "normalizer": None,
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": pattern}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False}]},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                  "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False, "ignore_merges": False,
                  "vocab": vocab, "merges": [[a, b] for a, b in merges]},
    }
    assert first == len(special_tokens)
    config = {}
    for key, names in (("eos_token", ("<|endoftext|>", "</s>", "<|eos|>")), ("bos_token", ("<s>", "<|bos|>")),
                       ("pad_token", ("<pad>", "<|pad|>"))):
        for n in names:
            if n in special_tokens:
                config[key] = n
                break
    return BpeTokenizer(spec, config)


# --------------------------------------------------------------------------------------------- WordPiece trainer
def train_wordpiece(texts: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = ("[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]"),
                    min_frequency: int = 2, lowercase: bool = False, prefix: str = "##") -> WordPieceTokenizer:
    """WordPiece vocabulary by pair merging: words are split into a first character and ``##`` continuations, and the
    pair with the largest count(ab) / (count(a) · count(b)) among those seen ``min_frequency`` times is merged
    (ties: the smaller pair), until the vocabulary is full. Writes the BertNormalizer / BertPreTokenizer layout."""
    specials = list(special_tokens)
    if "[UNK]" not in specials:
        specials = ["[UNK]"] + specials
    norm_spec = {"type": "BertNormalizer", "clean_text": True, "handle_chinese_chars": True, "strip_accents": None,
                 "lowercase": lowercase}
    normalize = build_normalizer(norm_spec)
    split, _ = build_pre_tokenizer({"type": "BertPreTokenizer"})
    counts: Counter = Counter()
    for t in texts:
        counts.update(split([normalize(t)]))
    vocab: Dict[str, int] = {}
    for s in specials:
        vocab.setdefault(s, len(vocab))
    words = [[w[0]] + [prefix + c for c in w[1:]] for w in counts]
    freqs = [counts[w] for w in counts]
    for sym in sorted({s for w in words for s in w}):
        vocab.setdefault(sym, len(vocab))
    unit: Counter = Counter()
    pairs: Counter = Counter()
    where: Dict[Tuple[str, str], set] = defaultdict(set)
    for k, (w, f) in enumerate(zip(words, freqs)):
        for s in w:
            unit[s] += f
        for a, b in zip(w, w[1:]):
            pairs[(a, b)] += f
            where[(a, b)].add(k)
    while len(vocab) < vocab_size:
        best, best_score = None, 0.0
        for (a, b), c in pairs.items():
            if c < min_frequency:
                continue
            score = c / (unit[a] * unit[b])
            if score > best_score or (score == best_score and best is not None and (a, b) < best):
                best, best_score = (a, b), score
        if best is None:
            break
        a, b = best
        merged = a + b[len(prefix):]
        vocab.setdefault(merged, len(vocab))
        for k in list(where.pop((a, b), ())):
            w, f = words[k], freqs[k]
            for s in w:
                unit[s] -= f
            for x, y in zip(w, w[1:]):
                pairs[(x, y)] -= f
                if pairs[(x, y)] <= 0:
                    del pairs[(x, y)]
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(merged)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            words[k] = out
            for s in out:
                unit[s] += f
            for x, y in zip(out, out[1:]):
                pairs[(x, y)] += f
                where[(x, y)].add(k)
        pairs.pop((a, b), None)
    spec = {
        "version": "1.0", "truncation": None, "padding": None,
        "added_tokens": [{"id": vocab[s], "content": s, "single_word": False, "lstrip": False, "rstrip": False,
                          "normalized": False, "special": True} for s in specials],
        "normalizer": norm_spec, "pre_tokenizer": {"type": "BertPreTokenizer"}, "post_processor": None,
        "decoder": {"type": "WordPiece", "prefix": prefix, "cleanup": True},
        "model": {"type": "WordPiece", "unk_token": "[UNK]", "continuing_subword_prefix": prefix,
                  "max_input_chars_per_word": 100, "vocab": vocab},
    }
    config = {k: v for k, v in (("pad_token", "[PAD]"), ("bos_token", "[CLS]"), ("eos_token", "[SEP]")) if v in specials}
    return WordPieceTokenizer(spec, config)
