"""File formats: safetensors, .ikw weights, .ikm packages, GGUF, PyTorch zip checkpoints, token files."""
from . import ikm, ikw, safetensors, tokens

__all__ = ["ikm", "ikw", "safetensors", "tokens"]
