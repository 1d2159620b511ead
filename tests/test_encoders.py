"""BERT and T5 against Hugging Face's implementations on random weights of tiny configurations."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from idrak_b200.models.encoder import BertEncoder, BertSpec, Seq2SeqGenerator, T5, T5Spec, relative_buckets  # noqa: E402


def test_bert_matches_hugging_face():
    torch.manual_seed(0)
    cfg = transformers.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                  max_position_embeddings=40, num_labels=1, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    ref = transformers.BertForSequenceClassification(cfg).eval()
    spec = BertSpec.from_hf_config(cfg.to_dict())
    assert spec.labels == 1 and spec.heads == 4
    m = BertEncoder(spec).eval()
    m.load_hf_tensors(ref.state_dict())
    ids = torch.randint(0, 100, (3, 12))
    mask = torch.ones(3, 12, dtype=torch.long)
    mask[1, 8:] = 0
    types = torch.zeros(3, 12, dtype=torch.long)
    types[:, 6:] = 1
    with torch.no_grad():
        want = ref(input_ids=ids, attention_mask=mask, token_type_ids=types, output_hidden_states=True)
        h = m.hidden(ids, mask, types)
        assert torch.allclose(h[mask.bool()], want.hidden_states[-1][mask.bool()], atol=1e-5)
        assert torch.allclose(m.classify(ids, mask, types), want.logits, atol=1e-5)
        e = m.embed(ids, mask)
    assert e.shape == (3, 32) and torch.allclose(e.norm(dim=-1), torch.ones(3), atol=1e-5)
    # padding does not change a row's vector
    assert torch.allclose(m.embed(ids[1:2, :8]), e[1:2], atol=1e-5)
    with pytest.raises(ValueError, match="positions"):
        m.hidden(torch.zeros(1, 41, dtype=torch.long))


@pytest.mark.parametrize("gated", [False, True])
def test_t5_matches_hugging_face_and_generates(gated):
    torch.manual_seed(1)
    cfg = transformers.T5Config(vocab_size=90, d_model=32, d_kv=8, d_ff=48, num_layers=2, num_decoder_layers=2, num_heads=4,
                                relative_attention_num_buckets=8, relative_attention_max_distance=20, dropout_rate=0.0,
                                feed_forward_proj="gated-gelu" if gated else "relu", tie_word_embeddings=not gated,
                                decoder_start_token_id=0)
    cfg.tie_word_embeddings = not gated
    ref = transformers.T5ForConditionalGeneration(cfg).eval()
    if gated:
        with torch.no_grad():
            ref.lm_head.weight = torch.nn.Parameter(torch.randn_like(ref.lm_head.weight) * 0.05)
            # an untied configuration leaves the two embedding tables on their own random values; released
            # checkpoints hold one shared table
            ref.encoder.embed_tokens.weight.copy_(ref.shared.weight)
            ref.decoder.embed_tokens.weight.copy_(ref.shared.weight)
    spec = T5Spec.from_hf_config(cfg.to_dict())
    assert spec.gated == gated and spec.tied_head == (not gated)
    m = T5(spec).eval()
    m.load_hf_tensors(ref.state_dict())
    ids = torch.randint(2, 90, (2, 11))
    mask = torch.ones(2, 11, dtype=torch.long)
    mask[1, 7:] = 0
    dec = torch.randint(2, 90, (2, 6))
    dec[:, 0] = 0
    with torch.no_grad():
        want = ref(input_ids=ids, attention_mask=mask, decoder_input_ids=dec).logits
        got = m(ids, dec, mask)
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
    labels = torch.randint(2, 90, (2, 6))
    labels[1, 4:] = -100
    with torch.no_grad():
        assert abs(m.loss(ids, labels, mask).item() - ref(input_ids=ids, attention_mask=mask, labels=labels).loss.item()) < 1e-4
        theirs = ref.generate(input_ids=ids, attention_mask=mask, max_new_tokens=8, do_sample=False)
    ours = Seq2SeqGenerator(m).generate(ids, mask, max_tokens=8)
    for row, want_row in zip(ours, theirs[:, 1:].tolist()):
        want_row = want_row[: want_row.index(1)] if 1 in want_row else [t for t in want_row if t != 0]
        assert [t for t in row if t != 0] == want_row
    sampled = Seq2SeqGenerator(m).generate(ids, mask, max_tokens=5, temperature=1.0, top_k=5, seed=3)
    assert sampled == Seq2SeqGenerator(m).generate(ids, mask, max_tokens=5, temperature=1.0, top_k=5, seed=3)


def test_relative_buckets():
    rel = torch.arange(-12, 13)[None]
    b = relative_buckets(rel, True, 8, 20)
    assert b.min() == 0 and b.max() == 7
    assert (b[0, :12] < 4).all() and (b[0, 13:] >= 4).all()         # the sign picks the half
    c = relative_buckets(rel, False, 8, 20)
    assert (c[0, 12:] == 0).all() and c[0, 0] == 6 and (c[0, :12].diff() <= 0).all()      # 4 + floor(4 log(12/4) / log(20/4))
