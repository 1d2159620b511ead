"""Finding and building tokenizers: a model folder, GGUF metadata, training from text.

Reference: PretrainedModel's tokenizer discovery (tokenizer.json, tokenizer.model, GGUF ``tokenizer.ggml.*`` keys:
src/Idrak/Models/PretrainedModel.cs, src/Idrak/Models/Gguf/GgufTokenizers.cs) and the trainers
(src/Idrak/Models/BpeTrainer.cs, Tokenizers/UnigramTrainer.cs, Tokenizers/WordPieceTrainer.cs).
"""
from __future__ import annotations

import json
import os
from typing import Iterable, Optional, Sequence

from .tokenizer import ByteTokenizer, HfTokenizer, SentencePieceTokenizer, Tokenizer


def _read_json(path: str) -> Optional[dict]:
    if not os.path.isfile(path):
        return None
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def load_tokenizer(folder: str) -> Tokenizer:
    """The tokenizer of a Hugging Face style model folder."""
    config = _read_json(os.path.join(folder, "tokenizer_config.json")) or {}
    gen = _read_json(os.path.join(folder, "generation_config.json")) or {}
    if not isinstance(config.get("chat_template"), str):
        for name in ("chat_template.jinja", "chat_template.json"):
            p = os.path.join(folder, name)
            if os.path.isfile(p):
                with open(p, "r", encoding="utf-8") as f:
                    text = f.read()
                config["chat_template"] = json.loads(text).get("chat_template") if name.endswith(".json") else text
                break
    tj = os.path.join(folder, "tokenizer.json")
    if os.path.isfile(tj):
        from .. import config as settings
        if settings.get("IDRAK_TOKENIZER") == "own":
            from .tokenizers_native import load_tokenizer_json
            t = load_tokenizer_json(tj, config)
            g = gen.get("eos_token_id")
            if g is not None:
                t.eos_token_ids = tuple(dict.fromkeys(list(t.eos_token_ids) + ([g] if isinstance(g, int) else list(g))))
            return t
        return HfTokenizer.from_file(tj, config, gen)
    tm = os.path.join(folder, "tokenizer.model")
    if os.path.isfile(tm):
        from .. import config as settings
        if settings.get("IDRAK_TOKENIZER") == "own":
            from .sentencepiece_model import load_sentencepiece
            t = load_sentencepiece(tm)          # this package's reader: no sentencepiece import
        else:
            t = SentencePieceTokenizer(tm, add_bos=bool(config.get("add_bos_token", True)))
        if isinstance(config.get("chat_template"), str):
            t.chat_template = config["chat_template"]
        return t
    vocab, merges = os.path.join(folder, "vocab.json"), os.path.join(folder, "merges.txt")
    if os.path.isfile(vocab) and os.path.isfile(merges):          # GPT-2 style pair of files
        from tokenizers import Tokenizer as _T, decoders, models, pre_tokenizers
        inner = _T(models.BPE.from_file(vocab, merges))
        inner.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        inner.decoder = decoders.ByteLevel()
        return HfTokenizer(inner, config, gen)
    raise FileNotFoundError(f"no tokenizer.json, tokenizer.model or vocab.json + merges.txt in {folder}")


def tokenizer_from_gguf(metadata: dict) -> Tokenizer:
    """Build the tokenizer a GGUF file carries in its ``tokenizer.ggml.*`` metadata (byte-level BPE: 'gpt2';
    SentencePiece-style vocabularies with scores: 'llama')."""
    from tokenizers import AddedToken, Tokenizer as _T, decoders, models, normalizers, pre_tokenizers
    kind = metadata.get("tokenizer.ggml.model")
    tokens = list(metadata.get("tokenizer.ggml.tokens") or [])
    if not tokens:
        raise ValueError("the GGUF file has no tokenizer.ggml.tokens")
    types = list(metadata.get("tokenizer.ggml.token_type") or [1] * len(tokens))
    vocab = {t: i for i, t in enumerate(tokens)}
    if kind == "gpt2":
        merges = [tuple(m.split(" ", 1)) for m in metadata.get("tokenizer.ggml.merges") or []]
        inner = _T(models.BPE(vocab, merges))
        inner.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        inner.decoder = decoders.ByteLevel()
    elif kind == "llama":
        scores = list(metadata.get("tokenizer.ggml.scores") or [0.0] * len(tokens))
        unk = int(metadata.get("tokenizer.ggml.unknown_token_id", 0))
        inner = _T(models.Unigram([(t, float(s)) for t, s in zip(tokens, scores)], unk_id=unk, byte_fallback=True))
        inner.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
        inner.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(),
                                           decoders.Strip(" ", 1, 0)])
    else:
        raise NotImplementedError(f"GGUF tokenizer model {kind!r}")
    special = [AddedToken(t, special=True) for t, ty in zip(tokens, types) if ty == 3]   # 3 = control
    if special:
        inner.add_special_tokens(special)

    def tok(key):
        i = metadata.get(key)
        return tokens[int(i)] if i is not None and 0 <= int(i) < len(tokens) else None

    config = {"bos_token": tok("tokenizer.ggml.bos_token_id"), "eos_token": tok("tokenizer.ggml.eos_token_id"),
              "pad_token": tok("tokenizer.ggml.padding_token_id"),
              "add_bos_token": bool(metadata.get("tokenizer.ggml.add_bos_token", kind == "llama")),
              "chat_template": metadata.get("tokenizer.chat_template")}
    return HfTokenizer(inner, config)


def train_tokenizer(kind: str, texts: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = (),
                    min_frequency: int = 2, byte_level: bool = True) -> HfTokenizer:
    """Train a 'bpe', 'unigram' or 'wordpiece' tokenizer on an iterator of strings."""
    from tokenizers import Tokenizer as _T, decoders, models, normalizers, pre_tokenizers, trainers
    specials = list(special_tokens)
    if kind == "bpe":
        inner = _T(models.BPE())
        if byte_level:
            inner.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            inner.decoder = decoders.ByteLevel()
            alphabet = pre_tokenizers.ByteLevel.alphabet()
        else:
            inner.pre_tokenizer = pre_tokenizers.Whitespace()
            alphabet = []
        trainer = trainers.BpeTrainer(vocab_size=vocab_size, min_frequency=min_frequency, special_tokens=specials,
                                      initial_alphabet=alphabet, show_progress=False)
    elif kind == "unigram":
        inner = _T(models.Unigram())
        inner.pre_tokenizer = pre_tokenizers.Metaspace()
        inner.decoder = decoders.Metaspace()
        trainer = trainers.UnigramTrainer(vocab_size=vocab_size, special_tokens=specials, unk_token="<unk>"
                                          if "<unk>" in specials else None, show_progress=False)
    elif kind == "wordpiece":
        if "[UNK]" not in specials:
            specials = ["[UNK]"] + specials
        inner = _T(models.WordPiece(unk_token="[UNK]"))
        inner.normalizer = normalizers.BertNormalizer(lowercase=False)
        inner.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
        inner.decoder = decoders.WordPiece()
        trainer = trainers.WordPieceTrainer(vocab_size=vocab_size, min_frequency=min_frequency,
                                            special_tokens=specials, show_progress=False)
    else:
        raise ValueError(f"unknown tokenizer kind {kind!r}: expected bpe, unigram or wordpiece")
    inner.train_from_iterator(texts, trainer)
    config = {}
    for key, names in (("eos_token", ("<|endoftext|>", "</s>", "<|eos|>", "[SEP]")), ("bos_token", ("<s>", "<|bos|>", "[CLS]")),
                       ("pad_token", ("<pad>", "<|pad|>", "[PAD]"))):
        for n in names:
            if n in specials:
                config[key] = n
                break
    return HfTokenizer(inner, config)
