"""Vision: ViT encoder / classifier over this package's kernels."""
from .vit import ImageClassifier, VisionTransformer, VitSpec

__all__ = ["ImageClassifier", "VisionTransformer", "VitSpec"]
