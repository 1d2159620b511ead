"""Model definitions: ``DecoderSpec`` and the decoder it builds; family registry in ``families``."""
from .spec import DecoderSpec, RopeSettings
from .decoder import Decoder, DecoderBlock, FeedForward, MixtureOfExperts, Norm, SelfAttention, build_decoder

__all__ = ["DecoderSpec", "RopeSettings", "Decoder", "DecoderBlock", "FeedForward", "MixtureOfExperts", "Norm",
           "SelfAttention", "build_decoder"]
