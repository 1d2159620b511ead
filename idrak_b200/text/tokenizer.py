"""Tokenizers: one small interface over the HF ``tokenizers`` runtime (BPE / Unigram / WordPiece from
``tokenizer.json``), SentencePiece ``.model`` files, vocabularies embedded in GGUF metadata, and a byte-level
fallback that needs no file. Trainers for BPE, Unigram and WordPiece wrap the same runtime.

The reference implements these tokenizer families itself (src/Idrak/Models/BpeTokenizer.cs, Tokenizers/UnigramTokenizer.cs,
Tokenizers/WordPieceTokenizer.cs and their trainers); here the battle-tested native runtime does the string work and
this module supplies loading rules, special-token bookkeeping and streaming decode.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Sequence


class Tokenizer:
    """encode / decode plus the special-token facts generation needs."""

    bos_token_id: Optional[int] = None
    eos_token_ids: Sequence[int] = ()
    pad_token_id: Optional[int] = None
    chat_template: Optional[str] = None
    special_tokens: Dict[str, int] = {}
    add_bos: bool = False

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        raise NotImplementedError

    def token_to_id(self, token: str) -> Optional[int]:
        return self.special_tokens.get(token)

    def stream(self, skip_special_tokens: bool = True) -> "StreamingDecoder":
        return StreamingDecoder(self, skip_special_tokens)


class StreamingDecoder:
    """Turns a growing token sequence into text pieces; holds back bytes of an unfinished UTF-8 character and
    re-decodes a short tail so pieces join exactly into ``decode(all ids)`` for prefix-stable decoders."""

    def __init__(self, tokenizer: Tokenizer, skip_special_tokens: bool = True, context: int = 6):
        self.tok, self.skip, self.context = tokenizer, skip_special_tokens, context
        self.ids: List[int] = []
        self.prefix_start = 0        # ids[prefix_start:read_to] were already emitted
        self.read_to = 0

    def push(self, token: int) -> str:
        self.ids.append(int(token))
        before = self.tok.decode(self.ids[self.prefix_start:self.read_to], self.skip)
        now = self.tok.decode(self.ids[self.prefix_start:], self.skip)
        if now.endswith("�") or len(now) < len(before):
            return ""                # an incomplete character: wait for the next token
        piece = now[len(before):]
        self.read_to = len(self.ids)
        self.prefix_start = max(self.read_to - self.context, self.prefix_start)
        return piece

    def flush(self) -> str:
        before = self.tok.decode(self.ids[self.prefix_start:self.read_to], self.skip)
        now = self.tok.decode(self.ids[self.prefix_start:], self.skip)
        self.read_to = len(self.ids)
        return now[len(before):] if len(now) >= len(before) else ""


class ByteTokenizer(Tokenizer):
    """UTF-8 bytes as ids 0..255, then the special tokens. For tests and models trained on raw bytes."""

    def __init__(self, specials: Sequence[str] = ("<|bos|>", "<|eos|>", "<|pad|>"), chat_template: Optional[str] = None):
        self.special_tokens = {s: 256 + i for i, s in enumerate(specials)}
        self._by_id = {v: k for k, v in self.special_tokens.items()}
        self.bos_token_id = self.special_tokens.get("<|bos|>")
        eos = self.special_tokens.get("<|eos|>")
        self.eos_token_ids = (eos,) if eos is not None else ()
        self.pad_token_id = self.special_tokens.get("<|pad|>")
        self.chat_template = chat_template

    @property
    def vocab_size(self) -> int:
        return 256 + len(self.special_tokens)

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        out: List[int] = []
        if add_special_tokens and self.add_bos and self.bos_token_id is not None:
            out.append(self.bos_token_id)
        i = 0
        while i < len(text):             # special tokens written in the text map to their ids
            hit = None
            if text[i] == "<":
                for s, v in self.special_tokens.items():
                    if text.startswith(s, i):
                        hit = (s, v)
                        break
            if hit:
                out.append(hit[1])
                i += len(hit[0])
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        parts: List[bytes] = []
        for t in ids:
            t = int(t)
            if t < 256:
                parts.append(bytes([t]))
            elif not skip_special_tokens and t in self._by_id:
                parts.append(self._by_id[t].encode())
        return b"".join(parts).decode("utf-8", errors="replace")


class HfTokenizer(Tokenizer):
    """A ``tokenizer.json`` run by the ``tokenizers`` library, with the neighbouring config files' special-token facts."""

    def __init__(self, inner, config: Optional[dict] = None, generation_config: Optional[dict] = None):
        self.inner = inner
        config = config or {}
        self.chat_template = config.get("chat_template") if isinstance(config.get("chat_template"), str) else None
        self.special_tokens = {t.content: i for i, t in inner.get_added_tokens_decoder().items() if t.special}

        def tid(key):
            v = config.get(key)
            if isinstance(v, dict):
                v = v.get("content")
            return inner.token_to_id(v) if isinstance(v, str) else None

        self.bos_token_id, self.pad_token_id = tid("bos_token"), tid("pad_token")
        eos = []
        g = (generation_config or {}).get("eos_token_id")
        if isinstance(g, int):
            eos.append(g)
        elif isinstance(g, list):
            eos += [int(x) for x in g]
        e = tid("eos_token")
        if e is not None and e not in eos:
            eos.append(e)
        self.eos_token_ids = tuple(eos)
        self.add_bos = bool(config.get("add_bos_token", False))

    @classmethod
    def from_file(cls, path: str, config: Optional[dict] = None, generation_config: Optional[dict] = None):
        from tokenizers import Tokenizer as _T
        return cls(_T.from_file(path), config, generation_config)

    @property
    def vocab_size(self) -> int:
        return self.inner.get_vocab_size(with_added_tokens=True)

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        return list(self.inner.encode(text, add_special_tokens=add_special_tokens).ids)

    def encode_batch(self, texts: Sequence[str], add_special_tokens: bool = True) -> List[List[int]]:
        return [list(e.ids) for e in self.inner.encode_batch(list(texts), add_special_tokens=add_special_tokens)]

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.inner.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def token_to_id(self, token: str) -> Optional[int]:
        return self.inner.token_to_id(token)

    def save(self, path: str) -> None:
        self.inner.save(path)


class SentencePieceTokenizer(Tokenizer):
    """A SentencePiece ``.model`` (Unigram or BPE) run by the ``sentencepiece`` library."""

    def __init__(self, model_file: str, add_bos: bool = True):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=model_file)
        self.add_bos = add_bos
        self.bos_token_id = self.sp.bos_id() if self.sp.bos_id() >= 0 else None
        self.eos_token_ids = (self.sp.eos_id(),) if self.sp.eos_id() >= 0 else ()
        self.pad_token_id = self.sp.pad_id() if self.sp.pad_id() >= 0 else None
        self.special_tokens = {self.sp.id_to_piece(i): i for i in range(self.sp.get_piece_size()) if self.sp.is_control(i)}

    @property
    def vocab_size(self) -> int:
        return self.sp.get_piece_size()

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids = list(self.sp.encode(text))
        if add_special_tokens and self.add_bos and self.bos_token_id is not None:
            ids.insert(0, self.bos_token_id)
        return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        ids = [int(i) for i in ids]
        if skip_special_tokens:
            ids = [i for i in ids if not self.sp.is_control(i)]
        return self.sp.decode(ids)
