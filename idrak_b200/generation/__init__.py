"""Generation: text generator over the serving engine, beam search, speculative decoding."""
from .text_generator import GenerationResult, TextGenerator

__all__ = ["GenerationResult", "TextGenerator"]
