import json

import pytest
import torch

from idrak_b200 import nn as inn
from idrak_b200.nn import losses


def test_builder_infers_sizes_and_round_trips_through_json():
    model = inn.Network.input(9).linear(64).relu().linear(32).relu().linear(1).build()
    assert [type(m).__name__ for m in model] == ["Linear", "ReLU", "Linear", "ReLU", "Linear"]
    assert model[2].in_features == 64 and model(torch.randn(5, 9)).shape == (5, 1)
    arch = json.loads(json.dumps(model.architecture))
    again = inn.Network.from_json(arch).build()
    again.load_state_dict(model.state_dict())
    x = torch.randn(4, 9)
    assert torch.equal(model(x), again(x)) and again.architecture == model.architecture

    cnn = (inn.Network.image(3, 32, 32).conv2d(8, 3, padding=1).batch_norm().relu().max_pool2d(2).conv2d(16, 3, stride=2, padding=1)
           .group_norm(4).gelu().upsample(2.0).adaptive_avg_pool2d(4).flatten().dropout(0.1).linear(10).softmax())
    assert cnn.output_shape == [10]
    m = cnn.build().eval()
    out = m(torch.randn(2, 3, 32, 32))
    assert out.shape == (2, 10) and torch.allclose(out.sum(-1), torch.ones(2), atol=1e-5)
    m2 = inn.Network.from_json(m.architecture).build().eval()
    m2.load_state_dict(m.state_dict())
    assert torch.allclose(m2(torch.ones(1, 3, 32, 32)), m(torch.ones(1, 3, 32, 32)))

    seq = (inn.Network.tokens(12).embedding(50, 16).positional().transformer(4, 32).transformer(4, 32, causal=True, norms="after")
           .lstm(8, sequences=True, bidirectional=True).gru(6))
    assert seq.output_shape == [6]
    assert seq.build()(torch.randint(0, 50, (3, 12))).shape == (3, 6)
    ts = inn.Network.sequence(20, 5).gru(7, sequences=True).layer_norm().attention(1).build()
    assert ts(torch.randn(2, 20, 5)).shape == (2, 20, 7)
    with pytest.raises(ValueError, match="images"):
        inn.Network.input(4).conv2d(3, 3)
    with pytest.raises(ValueError):
        inn.Network.from_json({"format": "other"})


def test_layer_types_describe_and_create():
    for module in (inn.Linear(4, 3, bias=False), inn.LayerNorm(8), inn.RMSNorm(8), inn.MultiHeadAttention(8, 2, causal=True),
                   inn.TransformerEncoderLayer(8, 2, 16, norms="after"), inn.Recurrent("gru", 4, 5, True, True, 2),
                   torch.nn.Conv2d(3, 4, (3, 5), stride=2, padding=1, dilation=2, groups=1), torch.nn.GELU(), torch.nn.GELU("tanh"),
                   torch.nn.MaxPool2d(2), torch.nn.Upsample(scale_factor=2.0, mode="bilinear", align_corners=False)):
        d = inn.describe(module)
        clone = inn.create(json.loads(json.dumps(d)))
        assert inn.describe(clone) == d, d
    nested = inn.Sequential(inn.Linear(2, 2), inn.Sequential(torch.nn.ReLU(), inn.Linear(2, 1)))
    d = inn.describe(nested)
    assert d["layers"][1]["layers"][1] == {"type": "linear", "in": 2, "out": 1, "bias": True}
    assert inn.create(d)(torch.zeros(1, 2)).shape == (1, 1)
    with pytest.raises(KeyError, match="no layer type"):
        inn.describe(torch.nn.Bilinear(2, 2, 2))
    with inn.LAYER_TYPES.register("mine", (torch.nn.Identity, lambda m: {}, lambda d: torch.nn.Identity())):
        assert inn.describe(torch.nn.Identity()) == {"type": "mine"}


def test_attention_layers_match_plain_statements():
    torch.manual_seed(0)
    mha = inn.MultiHeadAttention(16, 4, causal=True).eval()
    x = torch.randn(2, 7, 16)
    q, k, v = mha.qkv(x).view(2, 7, 3, 4, 4).unbind(2)
    s = torch.einsum("nthd,nshd->nhts", q, k) / 2.0
    s = s.masked_fill(~torch.ones(7, 7, dtype=torch.bool).tril(), float("-inf"))
    ref = mha.out(torch.einsum("nhts,nshd->nthd", s.softmax(-1), v).reshape(2, 7, 16))
    assert torch.allclose(mha(x), ref, atol=1e-5)
    pad = torch.zeros(2, 7, dtype=torch.bool)
    pad[1, 5:] = True
    enc = inn.TransformerEncoderLayer(16, 4, 32).eval()
    full, cut = enc(x, pad), enc(x[1:, :5])
    assert torch.allclose(full[1, :5], cut[0], atol=1e-5)          # padded keys do not leak into real positions
    ca = inn.CrossAttention(16, 4, memory_dim=12)
    assert ca(x, torch.randn(2, 9, 12)).shape == (2, 7, 16)
    wn = inn.weight_norm(inn.Linear(4, 3))
    assert wn(torch.randn(2, 4)).shape == (2, 3) and any("original" in n for n, _ in wn.named_parameters())


def test_losses():
    torch.manual_seed(1)
    logits, ids = torch.randn(6, 5), torch.randint(0, 5, (6,))
    onehot = torch.nn.functional.one_hot(ids, 5).float()
    assert torch.allclose(losses.cross_entropy(logits, onehot), losses.sparse_cross_entropy(logits, ids), atol=1e-6)
    assert torch.allclose(losses.cross_entropy(logits, onehot, 0.1), losses.sparse_cross_entropy(logits, ids, 0.1), atol=1e-6)
    assert torch.allclose(losses.token_log_probabilities(logits, ids).mean(), -losses.sparse_cross_entropy(logits, ids), atol=1e-6)
    assert losses.distillation_kl(logits, logits, 2.0).abs().item() < 1e-7
    t = torch.randn(6, 5)
    kl = losses.distillation_kl(logits, t, 2.0)
    ref = torch.nn.functional.kl_div(torch.log_softmax(logits / 2, -1), torch.softmax(t / 2, -1), reduction="batchmean") * 4
    assert torch.allclose(kl, ref, atol=1e-6)
    mask = torch.tensor([1, 1, 0, 0, 0, 0])
    assert torch.allclose(losses.distillation_kl(logits, t, 1.0, mask), losses.distillation_kl(logits[:2], t[:2]), atol=1e-6)
    p = torch.sigmoid(logits)
    assert torch.allclose(losses.binary_cross_entropy(p, onehot), losses.binary_cross_entropy_with_logits(logits, onehot), atol=1e-5)
    assert losses.mse(torch.ones(3), torch.zeros(3)).item() == 1.0 and losses.mae(torch.ones(3) * 2, torch.zeros(3)).item() == 2.0
    assert losses.pixel_cross_entropy(torch.randn(2, 4, 3, 3), torch.randint(0, 4, (2, 3, 3))).item() > 0
    lp = torch.randn(12, 2, 6).log_softmax(-1)
    c = losses.ctc(lp, torch.randint(1, 6, (2, 4)), torch.tensor([12, 12]), torch.tensor([4, 3]))
    assert c.item() > 0
    real, fake = [torch.ones(4) * 2], [-torch.ones(4) * 2]
    assert losses.hinge_discriminator(real, fake).item() == 0.0
    assert losses.least_squares_generator([torch.ones(3)]).item() == 0.0
    assert losses.feature_matching([[torch.ones(2, 2)]], [[torch.zeros(2, 2)]]).item() == 1.0


def test_relative_attention_flow_and_wavenet_layers():
    import torch
    from idrak_b200.nn import layers as L
    torch.manual_seed(0)
    att = L.RelativePositionAttention(32, 4, window=3)
    x = torch.randn(2, 9, 32)
    y = att(x, lengths=torch.tensor([9, 5]))
    assert y.shape == x.shape and torch.isfinite(y).all()
    # padded keys do not reach the kept positions of the short sequence
    x2 = x.clone()
    x2[1, 5:] = 7.0
    torch.testing.assert_close(att(x2, lengths=torch.tensor([9, 5]))[1, :5], y[1, :5])
    flow = L.AffineCoupling(8, hidden=16, layers=2, condition=4)
    with torch.no_grad():
        flow.post.weight.normal_(0, 0.1)
        flow.post.bias.normal_(0, 0.1)
    z = torch.randn(3, 8, 20)
    cond = torch.randn(3, 4, 20)
    mask = (torch.arange(20)[None, None, :] < torch.tensor([20, 12, 7])[:, None, None]).float()
    out, logdet = flow(z * mask, cond, mask)
    back = flow.reverse(out, cond, mask)
    torch.testing.assert_close(back, z * mask, rtol=1e-4, atol=1e-5)
    assert logdet.shape == (3,) and (out[:, :4] == (z * mask)[:, :4]).all()
    # the log-determinant is the one of the Jacobian: compare with autograd on one short sequence
    small = L.AffineCoupling(4, hidden=8, layers=1)
    with torch.no_grad():
        small.post.weight.normal_(0, 0.2)
    v = torch.randn(1, 4, 3)
    jac = torch.autograd.functional.jacobian(lambda t: small(t)[0].reshape(-1), v).reshape(12, 12)
    torch.testing.assert_close(torch.linalg.slogdet(jac)[1], small(v)[1][0], rtol=1e-4, atol=1e-5)
    for m in (att, flow, L.WaveNetBlock(6, 3, 2, 2)):
        twin = L.create(L.describe(m))
        assert type(twin) is type(m) and sum(p.numel() for p in twin.parameters()) == sum(p.numel() for p in m.parameters())
