"""A vision-language front end: an image encoder (ViT), a projector into the language model's width, and the decoder,
joined by placeholder tokens - every ``image_token`` in the text is replaced, in order, by one projected patch feature
of the images given with it (the layout LLaVA-style models use).

    vlm = VisionLanguageModel(vit, decoder, image_token=IMAGE_ID)
    ids = vlm.splice(text_ids, images=1)              # puts `patches` placeholders where the text has one image marker
    logits = vlm(pixels, ids)                         # pixels [n_images, C, S, S]
    loss = vlm.loss(pixels, ids, targets)             # targets: IGNORE at the placeholders

Training the projector alone (``vlm.trainable("projector")``) is the usual first stage; the encoder and the decoder
keep their weights.

Reference: the image-prefill path of the vision-language families (src/Idrak/Layers ImagePrefill; src/Idrak.Vision).
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import nn

from ..nn import layers as L


class VisionLanguageModel(nn.Module):
    def __init__(self, encoder, decoder, image_token: int, hidden: int = 0, use_class_token: bool = False):
        super().__init__()
        self.encoder, self.decoder = encoder, decoder
        self.image_token, self.use_class_token = int(image_token), use_class_token
        width_in, width_out = encoder.spec.dim, decoder.spec.dim
        hidden = hidden or width_out
        self.projector = nn.Sequential(L.Linear(width_in, hidden), nn.GELU(approximate="tanh"), L.Linear(hidden, width_out))

    @property
    def patches(self) -> int:
        """Placeholder tokens one image takes."""
        return self.encoder.spec.patches + (1 if self.use_class_token else 0)

    def splice(self, ids: Sequence[int], images: int = 1) -> List[int]:
        """Expand each of the first ``images`` image markers of ``ids`` into ``patches`` placeholders."""
        out, left = [], images
        for t in ids:
            if t == self.image_token and left > 0:
                out.extend([self.image_token] * self.patches)
                left -= 1
            else:
                out.append(int(t))
        if left:
            raise ValueError(f"the text has {images - left} image markers, {images} images were given")
        return out

    def image_features(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[n_images, C, S, S]`` -> ``[n_images * patches, decoder width]``."""
        h = self.encoder.hidden(pixels)
        if not self.use_class_token:
            h = h[:, 1:]
        return self.projector(h.reshape(-1, h.shape[-1]))

    def _embeds(self, pixels, ids):
        mask = ids == self.image_token
        if pixels is None:
            if bool(mask.any()):
                raise ValueError("the text has image placeholders but no images were given")
            return None
        return mask, self.image_features(pixels)

    def forward(self, pixels, ids: torch.Tensor, positions=None) -> torch.Tensor:
        return self.decoder(ids, positions, embeds=self._embeds(pixels, ids))

    def loss(self, pixels, ids: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
        return self.decoder.loss(ids, targets, ignore_index=ignore_index, embeds=self._embeds(pixels, ids))

    def trainable(self, *parts: str) -> List[nn.Parameter]:
        """Freeze everything but the named parts ("projector", "decoder", "encoder") and return what is left trainable."""
        out = []
        for name in ("encoder", "decoder", "projector"):
            for p in getattr(self, name).parameters():
                p.requires_grad_(name in parts)
                if name in parts:
                    out.append(p)
        return out
