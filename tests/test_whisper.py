"""Whisper against the transformers implementation on a random-initialised tiny configuration: encoder output, logits,
incremental decoding and greedy generation; and the feature extractor's shape and scaling."""
import pytest
import torch

from idrak_b200.audio.whisper import Whisper, WhisperSpec, features, sinusoids

transformers = pytest.importorskip("transformers")


def _pair():
    from transformers import WhisperConfig, WhisperForConditionalGeneration
    torch.manual_seed(0)
    cfg = WhisperConfig(vocab_size=120, num_mel_bins=16, d_model=32, encoder_layers=2, decoder_layers=2,
                        encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64,
                        max_source_positions=50, max_target_positions=24, pad_token_id=0, bos_token_id=1, eos_token_id=2,
                        decoder_start_token_id=1, suppress_tokens=None, begin_suppress_tokens=None)
    theirs = WhisperForConditionalGeneration(cfg).eval()
    mine = Whisper(WhisperSpec.from_hf_config(cfg.to_dict())).eval()
    missing = mine.load_hf(theirs.state_dict())
    assert missing == []
    return mine, theirs


def test_logits_match_transformers():
    mine, theirs = _pair()
    mel = torch.randn(2, 16, 100)
    ids = torch.randint(3, 120, (2, 7))
    with torch.no_grad():
        want = theirs(input_features=mel, decoder_input_ids=ids)
        got_audio = mine.encode(mel)
        got = mine(mel, ids)
    torch.testing.assert_close(got_audio, want.encoder_last_hidden_state, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got, want.logits, rtol=1e-4, atol=1e-4)
    # incremental decoding gives the same last-position logits as the full pass
    cross = mine.cross_keys_values(got_audio)
    caches = [dict() for _ in mine.decoder]
    with torch.no_grad():
        mine.decode(ids[:, :4], cross, caches)
        step = None
        for t in range(4, 7):
            step = mine.decode(ids[:, t:t + 1], cross, caches, offset=t)
    torch.testing.assert_close(step[:, 0], got[:, -1], rtol=1e-4, atol=1e-4)


def test_greedy_generation_matches_transformers():
    mine, theirs = _pair()
    mel = torch.randn(2, 16, 100)
    got = mine.generate(mel, prefix=[1], end_token=2, max_tokens=12)
    with torch.no_grad():
        want = theirs.generate(input_features=mel, max_new_tokens=12, do_sample=False, num_beams=1)
    for mine_ids, row in zip(got, want.tolist()):
        tail = [t for t in row[1:] if t != 2 and t != 0][: len(mine_ids)]
        assert mine_ids[: len(tail)] == tail and len(mine_ids) >= min(len(tail), 1)


def test_features_and_positions():
    x = torch.sin(torch.arange(16000 * 2) * 2 * 3.14159 * 440 / 16000)
    f = features(x, mels=80)
    assert f.shape == (80, 3000) and f.max() <= 2.0 and (f.max() - f.min()) <= 2.0 + 1e-5      # 8 decades / 4
    assert f[:, 2500:].std() < 1e-6                                                           # the padded tail is flat
    p = sinusoids(50, 32)
    assert p.shape == (50, 32) and torch.allclose(p[0, :16], torch.zeros(16)) and torch.allclose(p[0, 16:], torch.ones(16))
