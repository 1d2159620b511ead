"""The vision-language front end: placeholders are replaced by projected patch features in order, text-only input is
the plain decoder, and the projector learns a task the text alone cannot solve."""
import pytest
import torch

from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.vision import VisionTransformer, VitSpec
from idrak_b200.vision.vlm import VisionLanguageModel

IMG = 99


def _pair(seed=0):
    torch.manual_seed(seed)
    vit = VisionTransformer(VitSpec(image_size=16, patch_size=8, channels=1, dim=32, layers=1, heads=2, ff_dim=64, classes=2))
    dec = build_decoder(DecoderSpec.llama(layers=2, dim=48, heads=4, kv_heads=4, ff_dim=96, vocab=100, max_positions=64), seed=1).float()
    return VisionLanguageModel(vit, dec, image_token=IMG)


def test_splice_and_replacement_order():
    vlm = _pair()
    assert vlm.patches == 4
    ids = vlm.splice([5, IMG, 6, 7], images=1)
    assert ids == [5, IMG, IMG, IMG, IMG, 6, 7]
    with pytest.raises(ValueError, match="image markers"):
        vlm.splice([5, 6], images=1)
    t = torch.tensor([ids])
    px = torch.randn(1, 1, 16, 16)
    feats = vlm.image_features(px)
    assert feats.shape == (4, 48)
    # the decoder sees exactly those rows at the placeholder positions
    seen = {}
    hook = vlm.decoder.blocks[0].register_forward_pre_hook(lambda m, a: seen.setdefault("x", a[0].detach().clone()))
    vlm(px, t)
    hook.remove()
    torch.testing.assert_close(seen["x"][0, 1:5], feats.detach(), rtol=1e-5, atol=1e-6)
    # text without placeholders is the plain decoder; placeholders without images are refused
    plain = torch.tensor([[5, 6, 7, 8]])
    torch.testing.assert_close(vlm(None, plain), vlm.decoder(plain))
    with pytest.raises(ValueError, match="no images"):
        vlm(None, t)
    with pytest.raises(ValueError, match="positions are marked"):
        vlm(torch.randn(2, 1, 16, 16), t)


def test_model_learns_to_name_the_bright_half_from_the_image_alone():
    vlm = _pair(1)
    params = vlm.trainable("projector")
    assert all(not p.requires_grad for p in vlm.decoder.parameters()) and len(params) == 4
    params = vlm.trainable("projector", "decoder")                         # the encoder stays frozen
    assert all(not p.requires_grad for p in vlm.encoder.parameters())
    opt = torch.optim.Adam(params, lr=5e-3)
    g = torch.Generator().manual_seed(2)
    ids = torch.tensor([vlm.splice([IMG, 10], images=1)] * 16)              # "<image> which?" -> answer token
    targets = torch.full_like(ids, -100)
    first = None
    for step in range(80):
        side = torch.randint(0, 2, (16,), generator=g)
        px = 0.1 * torch.randn(16, 1, 16, 16, generator=g)
        for n in range(16):
            px[n, 0, :, (8 if side[n] else 0):(16 if side[n] else 8)] += 1.0
        targets[:, -1] = 20 + side                                           # token 20: left half bright, 21: right
        loss = vlm.loss(px, ids, targets)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = float(loss.detach()) if first is None else first
    assert float(loss.detach()) < 0.3 < first              # the text is the same for both answers: only the image tells
