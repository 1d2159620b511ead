"""The package's own BPE / WordPiece / Unigram runtimes against the `tokenizers` library on the same tokenizer.json,
the native merge engine against the Python merge loop, and the BPE trainer's round trip."""
import json
import os

import pytest

from idrak_b200 import _native
from idrak_b200.text.tokenizers_native import (BpeTokenizer, UnigramTokenizer, WordPieceTokenizer, bytes_to_unicode,
                                               load_tokenizer_json, train_bpe)

tokenizers = pytest.importorskip("tokenizers")

CORPUS = [
    "The quick brown fox jumps over the lazy dog.",
    "Pack my box with five dozen liquor jugs!",
    "def fib(n):\n    return n if n < 2 else fib(n - 1) + fib(n - 2)\n",
    "Tokenizers split text into pieces; pieces become numbers, numbers become vectors.",
    "It's 2024 and we've got 3 cats, 12 dogs and 1,000 fish.",
    "naïve café résumé coöperate – “quotes” and ellipsis…",
    "東京は日本の首都です。 Привет, мир! مرحبا بالعالم",
    "    indented\ttabs and   runs   of   spaces  \n\n",
] * 6
PROBES = [
    "Hello world, the quick brown fox isn't lazy.",
    "numbers 1234567 and code: x = fib(10) + 3",
    "unicode: café 東京 Привет 🙂 emoji",
    "  leading spaces and trailing   ",
    "",
    "a",
    "I've we'll they're don't",
]


def _train(kind, tmp_path):
    from idrak_b200.text.tokenizer_io import train_tokenizer
    specials = {"bpe": ["<|endoftext|>"], "wordpiece": ["[UNK]", "[CLS]", "[SEP]", "[PAD]"], "unigram": ["<unk>", "</s>"]}[kind]
    tok = train_tokenizer(kind, CORPUS, 400, specials, min_frequency=1)
    path = os.path.join(tmp_path, f"{kind}.json")
    tok.inner.save(path)
    return tok.inner, path


def test_byte_table_is_a_bijection():
    t = bytes_to_unicode()
    assert len(t) == 256 and len(set(t.values())) == 256
    assert t[ord("A")] == "A" and t[ord(" ")] == "Ġ"


def test_bpe_matches_library(tmp_path):
    ref, path = _train("bpe", tmp_path)
    own = load_tokenizer_json(path)
    assert isinstance(own, BpeTokenizer)
    for text in PROBES + CORPUS[:8]:
        assert own.encode(text) == ref.encode(text, add_special_tokens=False).ids, text
        assert own.decode(own.encode(text)) == text
    ids = own.encode("one<|endoftext|>two")
    assert own.special_tokens["<|endoftext|>"] in ids
    assert own.decode(ids) == "onetwo" and own.decode(ids, skip_special_tokens=False) == "one<|endoftext|>two"


@pytest.mark.skipif(not _native.available(), reason="native library not built")
def test_native_merge_engine_matches_python_loop(tmp_path):
    _, path = _train("bpe", tmp_path)
    own = load_tokenizer_json(path)
    assert own.native
    words = own.pre_tokenize([" ".join(CORPUS[:8])])
    fast = own._encode_words(words)
    again = own._encode_words(words)              # second pass is served from the engine's cache
    slow = [i for w in words for i in own._merge_python(own._symbols(w))]
    assert fast == slow == again


def test_wordpiece_matches_library(tmp_path):
    ref, path = _train("wordpiece", tmp_path)
    own = load_tokenizer_json(path)
    assert isinstance(own, WordPieceTokenizer)
    for text in PROBES[:4] + CORPUS[:6]:
        assert own.encode(text) == ref.encode(text, add_special_tokens=False).ids, text
    assert own.decode(own.encode("the quick brown fox.")) == ref.decode(ref.encode("the quick brown fox.").ids)


def test_unigram_matches_library(tmp_path):
    ref, path = _train("unigram", tmp_path)
    own = load_tokenizer_json(path)
    assert isinstance(own, UnigramTokenizer)
    for text in PROBES[:2] + PROBES[3:] + CORPUS[:5]:
        assert own.encode(text) == ref.encode(text, add_special_tokens=False).ids, text
    t = "The quick brown fox"
    assert own.decode(own.encode(t)) == t


def test_bpe_trainer_round_trip(tmp_path):
    tok = train_bpe(CORPUS, 420, special_tokens=["<|endoftext|>"], min_frequency=2)
    assert tok.vocab_size <= 420 and tok.vocab_size > 257
    assert tok.eos_token_ids == (0,)
    text = "The quick brown fox jumps over numbers 12 and café."
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    assert len(ids) < len(text.encode("utf-8")) * 0.7            # the merges compress
    path = os.path.join(tmp_path, "own.json")
    tok.save(path)
    lib = tokenizers.Tokenizer.from_file(path)                      # the library reads what the trainer wrote
    assert lib.encode(text, add_special_tokens=False).ids == ids
    again = load_tokenizer_json(path)
    assert again.encode(text) == ids


def test_unsupported_parts_are_refused_by_name(tmp_path):
    spec = {"model": {"type": "BPE", "vocab": {"a": 0}, "merges": []}, "pre_tokenizer": {"type": "CharDelimiterSplit"}}
    p = os.path.join(tmp_path, "t.json")
    json.dump(spec, open(p, "w"))
    with pytest.raises(ValueError, match="CharDelimiterSplit"):
        load_tokenizer_json(p)


def test_wordpiece_trainer_round_trip(tmp_path):
    from idrak_b200.text.tokenizers_native import train_wordpiece
    tok = train_wordpiece(CORPUS, 300, min_frequency=2, lowercase=True)
    assert 100 < tok.vocab_size <= 300 and tok.pad_token_id == tok.vocab["[PAD]"]
    text = "the quick brown fox jumps over the lazy dog."
    ids = tok.encode(text)
    assert tok.unk_id not in ids and tok.decode(ids) == text
    assert len(ids) < len(text.replace(" ", ""))                     # pieces longer than single characters were learned
    assert any(t.startswith("##") and len(t) > 3 for t in tok.vocab)
    path = os.path.join(tmp_path, "wp.json")
    tok.save(path)
    lib = tokenizers.Tokenizer.from_file(path)
    assert lib.encode(text, add_special_tokens=False).ids == ids      # the library reads the file and agrees
    assert tok.encode("zzzq ☃") .count(tok.unk_id) >= 1             # a symbol never seen is unknown
