"""Generation: text generator over the serving engine, beam search, speculative decoding."""
from .beam import BeamSearch, Hypothesis
from .speculative import SpeculativeDecoder, SpeculativeResult
from .text_generator import GenerationResult, TextGenerator

__all__ = ["BeamSearch", "Hypothesis", "SpeculativeDecoder", "SpeculativeResult", "GenerationResult", "TextGenerator"]
