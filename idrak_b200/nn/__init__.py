"""General layers, the JSON-describable network builder and losses."""
from . import losses
from .builder import Network, NetworkBuilder
from .layers import (LAYER_TYPES, CrossAttention, Embedding, GlobalAveragePool2d, LayerNorm, Linear, MultiHeadAttention,
                     PositionalEncoding, QuickGELU, Recurrent, RMSNorm, Sequential, TransformerEncoderLayer, create, describe,
                     weight_norm)
