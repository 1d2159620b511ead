"""ViT parity with transformers on a tiny random model (CPU), and the classifier wrapper."""
import pytest
import torch

from idrak_b200.vision import ImageClassifier, VisionTransformer, VitSpec


def test_vit_matches_transformers():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.ViTConfig(image_size=32, patch_size=8, num_channels=3, hidden_size=64, num_hidden_layers=2,
                                 num_attention_heads=4, intermediate_size=128, num_labels=5)
    torch.manual_seed(0)
    ref = transformers.ViTForImageClassification(cfg).eval()
    spec = VitSpec.from_hf_config(cfg.to_dict())
    assert spec.patches == 16 and spec.classes == 5
    mine = VisionTransformer(spec).float().eval()
    mine.load_hf_tensors(ref.state_dict())
    x = torch.randn(3, 3, 32, 32)
    with torch.no_grad():
        want = ref(pixel_values=x).logits
        got = mine(x)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    imgs = torch.randint(0, 256, (2, 40, 50, 3), dtype=torch.uint8)
    out = ImageClassifier(mine, labels=list("abcde")).classify(imgs, k=3)
    assert len(out) == 2 and len(out[0]) == 3 and out[0][0]["probability"] >= out[0][1]["probability"]
    assert set(o["label"] for o in out[0]) <= set("abcde")
    e = mine.embed(mine.preprocess(imgs))
    assert e.shape == (2, 64) and torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-5)
