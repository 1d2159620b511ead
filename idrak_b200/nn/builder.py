"""Fluent network builder with JSON round-trip: every step adds one layer whose input size comes from the previous
layer's output shape, ``build()`` returns an ordinary ``Sequential``, ``to_json()`` writes the recipe and
``Network.from_json`` replays it.

    model = Network.input(9).linear(64).relu().linear(32).relu().linear(1).build()
    model = Network.image(3, 32, 32).conv2d(16, 3, padding=1).relu().max_pool2d(2).flatten().linear(10).build()
    same = Network.from_json(model.architecture).build()

Reference: Network / NetworkBuilder (src/Idrak/Layers/NetworkBuilder.cs: input kinds features / image / tokens /
sequence, one method per layer, ToJson / FromJson, ArchitectureOf).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch
from torch import nn

from . import layers as L

INPUT_KINDS = ("features", "image", "tokens", "sequence")


class NetworkBuilder:
    def __init__(self, kind: str, shape: Sequence[int]):
        if kind not in INPUT_KINDS:
            raise ValueError(f"input kind must be one of {', '.join(INPUT_KINDS)}")
        if any(int(v) <= 0 for v in shape):
            raise ValueError("sizes must be positive")
        self.kind, self.input_shape = kind, [int(v) for v in shape]
        self.shape: List[int] = list(self.input_shape)           # shape of one sample after the layers so far
        self.steps: List[dict] = []
        self.modules: List[nn.Module] = []

    # ------------------------------------------------------------------ plumbing
    def _add(self, description: dict) -> "NetworkBuilder":
        module = L.create(description)
        probe = torch.zeros(2, *self.shape, dtype=torch.long if (self.kind == "tokens" and not self.modules) else torch.float32)
        was = module.training
        module.eval()
        with torch.no_grad():
            out = module(probe)
        module.train(was)
        self.shape = list(out.shape[1:])
        self.steps.append(description)
        self.modules.append(module)
        return self

    def _features(self) -> int:
        return self.shape[-1]

    def _channels(self) -> int:
        if len(self.shape) != 3:
            raise ValueError(f"this layer takes images [N, C, H, W]; the network so far gives {['N'] + self.shape}")
        return self.shape[0]

    # ------------------------------------------------------------------ layers
    def linear(self, out: int, bias: bool = True):
        return self._add({"type": "linear", "in": self._features(), "out": out, "bias": bias})

    def embedding(self, vocabulary: int, dim: int):
        return self._add({"type": "embedding", "vocabulary": vocabulary, "dim": dim})

    def positional(self, max_length: Optional[int] = None):
        return self._add({"type": "positional", "maxLength": max_length or self.shape[0], "dim": self._features()})

    def layer_norm(self, epsilon: float = 1e-5):
        return self._add({"type": "layernorm", "features": self._features(), "epsilon": epsilon})

    def rms_norm(self, epsilon: float = 1e-6):
        return self._add({"type": "rmsnorm", "features": self._features(), "epsilon": epsilon})

    def attention(self, heads: int, causal: bool = False):
        return self._add({"type": "attention", "dim": self._features(), "heads": heads, "causal": causal})

    def transformer(self, heads: int, ff_dim: int, causal: bool = False, norms: str = "before"):
        d = {"type": "transformer", "dim": self._features(), "heads": heads, "ffDim": ff_dim, "causal": causal}
        if norms == "after":
            d["norms"] = "after"
        return self._add(d)

    def lstm(self, hidden: int, sequences: bool = False, bidirectional: bool = False, layers: int = 1):
        return self._recurrent("lstm", hidden, sequences, bidirectional, layers)

    def gru(self, hidden: int, sequences: bool = False, bidirectional: bool = False, layers: int = 1):
        return self._recurrent("gru", hidden, sequences, bidirectional, layers)

    def _recurrent(self, kind, hidden, sequences, bidirectional, layers):
        d = {"type": kind, "in": self._features(), "hidden": hidden, "sequences": sequences}
        if bidirectional:
            d["bidirectional"] = True
        if layers != 1:
            d["layers"] = layers
        return self._add(d)

    def conv2d(self, out: int, kernel: Union[int, Tuple[int, int]], stride=1, padding=0, dilation=1, groups: int = 1, bias: bool = True):
        d = {"type": "conv2d", "in": self._channels(), "out": out, "kernel": list(L._pair(kernel)), "stride": list(L._pair(stride)),
             "padding": list(L._pair(padding)), "bias": bias}
        if L._pair(dilation) != (1, 1):
            d["dilation"] = list(L._pair(dilation))
        if groups != 1:
            d["groups"] = groups
        return self._add(d)

    def conv_transpose2d(self, out: int, kernel, stride=1, padding=0, output_padding=0, bias: bool = True):
        return self._add({"type": "convtranspose2d", "in": self._channels(), "out": out, "kernel": list(L._pair(kernel)),
                          "stride": list(L._pair(stride)), "padding": list(L._pair(padding)),
                          "outputPadding": list(L._pair(output_padding)), "dilation": [1, 1], "groups": 1, "bias": bias})

    def batch_norm(self, momentum: float = 0.1, epsilon: float = 1e-5):
        return self._add({"type": "batchnorm", "channels": self._channels(), "momentum": momentum, "epsilon": epsilon})

    def group_norm(self, groups: int, epsilon: float = 1e-5, affine: bool = True):
        return self._add({"type": "groupnorm", "groups": groups, "channels": self._channels(), "epsilon": epsilon, "affine": affine})

    def max_pool2d(self, kernel, stride=None, padding=0):
        return self._add({"type": "maxpool2d", "kernel": list(L._pair(kernel)), "stride": list(L._pair(stride or kernel)),
                          "padding": list(L._pair(padding))})

    def avg_pool2d(self, kernel, stride=None, padding=0, count_include_pad: bool = True):
        return self._add({"type": "avgpool2d", "kernel": list(L._pair(kernel)), "stride": list(L._pair(stride or kernel)),
                          "padding": list(L._pair(padding)), "countIncludePad": count_include_pad})

    def adaptive_avg_pool2d(self, size):
        return self._add({"type": "adaptiveavgpool2d", "size": list(L._pair(size))})

    def adaptive_max_pool2d(self, size):
        return self._add({"type": "adaptivemaxpool2d", "size": list(L._pair(size))})

    def upsample(self, scale=None, size=None, mode: str = "nearest"):
        d = {"type": "upsample", "mode": mode, "alignCorners": False}
        if size is not None:
            d["size"] = list(L._pair(size))
        else:
            d["scale"] = [float(v) for v in L._scale(scale or 2.0)]
        return self._add(d)

    def global_avg_pool2d(self):
        return self._add({"type": "globalavgpool2d"})

    def flatten(self):
        return self._add({"type": "flatten"})

    def dropout(self, p: float = 0.5):
        return self._add({"type": "dropout", "p": p})

    def relu(self):
        return self._add({"type": "relu"})

    def tanh(self):
        return self._add({"type": "tanh"})

    def sigmoid(self):
        return self._add({"type": "sigmoid"})

    def gelu(self, exact: bool = False):
        return self._add({"type": "gelu_exact" if exact else "gelu"})

    def quick_gelu(self):
        return self._add({"type": "quick_gelu"})

    def softmax(self):
        return self._add({"type": "softmax"})

    def layer(self, description: dict):
        """Any registered layer type by its description."""
        return self._add(dict(description))

    # ------------------------------------------------------------------ results
    @property
    def output_shape(self) -> List[int]:
        return list(self.shape)

    def to_json(self) -> dict:
        return {"format": "idrak-network/1", "input": {"kind": self.kind, "shape": list(self.input_shape)},
                "layers": [dict(s) for s in self.steps]}

    def build(self) -> L.Sequential:
        model = L.Sequential(*self.modules)
        model.architecture = self.to_json()
        return model


class Network:
    @staticmethod
    def input(features: int) -> NetworkBuilder:
        return NetworkBuilder("features", [features])

    @staticmethod
    def image(channels: int, height: int, width: int) -> NetworkBuilder:
        return NetworkBuilder("image", [channels, height, width])

    @staticmethod
    def tokens(length: int) -> NetworkBuilder:
        return NetworkBuilder("tokens", [length])

    @staticmethod
    def sequence(length: int, features: int) -> NetworkBuilder:
        return NetworkBuilder("sequence", [length, features])

    @staticmethod
    def from_json(description: dict) -> NetworkBuilder:
        if description.get("format") != "idrak-network/1":
            raise ValueError("not a network description (format 'idrak-network/1')")
        b = NetworkBuilder(description["input"]["kind"], description["input"]["shape"])
        for step in description["layers"]:
            b.layer(step)
        return b

    @staticmethod
    def architecture_of(model: nn.Module):
        arch = getattr(model, "architecture", None)
        return None if arch is None else {**arch, "layers": [dict(s) for s in arch["layers"]]}
