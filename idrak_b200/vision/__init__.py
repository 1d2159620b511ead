"""Vision: ViT encoder / classifier, an anchor-free detector and a U-shaped segmenter over this package's kernels, box
utilities and detection metrics."""
from .models import CenterDetector, Segmenter, mean_iou
from .vit import ImageClassifier, VisionTransformer, VitSpec

__all__ = ["CenterDetector", "ImageClassifier", "Segmenter", "VisionTransformer", "VitSpec", "mean_iou"]
