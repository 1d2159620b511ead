"""SentencePiece model files, the precompiled character map and Unigram training, with no sentencepiece import on the
tested path (the installed library is used only as an oracle where present)."""
import random

import pytest

from idrak_b200.text import sentencepiece_model as spm
from idrak_b200.text.unigram_trainer import train_unigram, train_unigram_pieces

CORPUS = [("the quick brown fox jumps over the lazy dog . a tokenizer learns pieces from text . unigram models keep the "
           "pieces that explain the corpus best . tokenization tokenizers tokenized . ") * 4,
          "learning learned learner relearn the theory of thermodynamics and the thermal theorem",
          "naïve café façade über straße"]


def test_double_array_trie_agrees_with_a_dictionary():
    rnd = random.Random(3)
    keys = {bytes(rnd.randint(1, 255) for _ in range(rnd.randint(1, 6))): i for i in range(2000)}
    t = spm.DoubleArrayTrie.build(keys)
    again = spm.DoubleArrayTrie(list(__import__("struct").unpack(f"<{len(t.units)}I", t.to_bytes())))
    for _ in range(5000):
        k = bytes(rnd.randint(1, 255) for _ in range(rnd.randint(1, 6)))
        assert again.lookup(k) == keys.get(k)
        want = sorted((keys[k[:n]], n) for n in range(1, len(k) + 1) if k[:n] in keys)
        assert sorted(again.common_prefixes(k)) == want
    assert all(again.lookup(k) == v for k, v in keys.items())
    with pytest.raises(ValueError):
        spm.DoubleArrayTrie.build({b"a\0b": 1})


def test_precompiled_normalizer_replaces_longest_match_and_copies_the_rest():
    n = spm.PrecompiledNormalizer.from_rules({"ﬁ": "fi", "Ａ": "A", "　": " ", "ab": "X", "abc": "Y"})
    assert n("ﬁne Ａ　x") == "fine A x"
    assert n("abcab-a") == "YX-a"
    assert n("日本語 🙂") == "日本語 🙂"
    assert spm.PrecompiledNormalizer(n.raw)("Ａ") == "A"            # survives its byte form
    assert spm.PrecompiledNormalizer(b"")("same") == "same"
    with pytest.raises(ValueError):
        spm.PrecompiledNormalizer(b"\xff\xff\xff\x7f1234")


def test_model_file_round_trip_and_tokenizer():
    pieces = train_unigram_pieces(CORPUS, 90)
    model = spm.from_unigram(pieces, byte_fallback=True, rules={"Ａ": "A"})
    data = spm.write_model(model)
    back = spm.read_model(data)
    assert back.pieces == model.pieces and back.types == model.types and back.byte_fallback
    assert all(abs(a - b) <= 1e-6 * max(1.0, abs(a)) for a, b in zip(back.scores, model.scores))      # stored as float32
    assert (back.unk_id, back.bos_id, back.eos_id, back.pad_id) == (0, 1, 2, -1)
    assert back.precompiled_charsmap == model.precompiled_charsmap and back.add_dummy_prefix
    tok = spm.to_tokenizer(back)
    text = "the tokenizer learns Ａ pieces 🙂"
    ids = tok.encode(text)
    assert tok.decode(ids) == "the tokenizer learns A pieces 🙂"       # normalised; the emoji went through byte pieces
    assert any(tok.id_to_token[i].startswith("<0x") for i in ids)
    assert tok.bos_token_id == 1 and tok.eos_token_ids == (2,)
    with pytest.raises(ValueError):
        spm.read_model(b"\x08\x01")


def test_unigram_training_gives_a_vocabulary_that_compresses_and_round_trips():
    tok = train_unigram(CORPUS, 120)
    assert tok.vocab_size <= 120 and tok.vocab_size > 40
    vocab = set(tok.vocab)
    assert "▁the" in vocab and "▁pieces" in vocab
    assert all(ch in vocab for ch in "abcdefghijklmnopqrstuvwxyz."), "every seen character stays a piece"
    for text in ("the lazy tokenizer explains the theory", "unseen wordforms relearned", "über café"):
        ids = tok.encode(text)
        assert tok.decode(ids) == text
    seen = "the lazy tokenizer learns pieces from the corpus"
    assert len(tok.encode(seen)) < len(seen) * 0.4
    assert train_unigram_pieces(CORPUS, 120) == train_unigram_pieces(CORPUS, 120)          # deterministic
    with pytest.raises(ValueError):
        train_unigram_pieces(CORPUS, 5)


def test_scores_are_log_probabilities():
    import math
    pieces = train_unigram_pieces(CORPUS, 100)
    assert abs(sum(math.exp(s) for _, s in pieces) - 1.0) < 1e-6
    assert pieces == sorted(pieces, key=lambda ps: (-ps[1], ps[0]))


def test_reader_agrees_with_the_sentencepiece_library_when_it_is_installed(tmp_path):
    sp = pytest.importorskip("sentencepiece")
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(CORPUS * 3))
    prefix = str(tmp_path / "m")
    sp.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=100, model_type="unigram",
                                  hard_vocab_limit=False, minloglevel=2)
    oracle = sp.SentencePieceProcessor(model_file=prefix + ".model")
    model = spm.read_model(prefix + ".model")
    assert model.pieces == [oracle.id_to_piece(i) for i in range(oracle.get_piece_size())]
    assert model.precompiled_charsmap, "the default nmt_nfkc map is present"
    tok = spm.to_tokenizer(model)
    for text in ("the quick brown tokenizer", "ｆｕｌｌｗｉｄｔｈ text  with   spaces", "thermal theory of pieces ."):
        assert tok.encode(text) == oracle.encode(text), text
        assert tok.decode(tok.encode(text)) == oracle.decode(oracle.encode(text))
