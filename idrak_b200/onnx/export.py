"""Write networks as ONNX (opset 17). Works layer by layer on ``Sequential`` models made of this package's layers and
the common library layers; each layer adds its nodes and initialisers to a graph writer.

    data = export(model, input_shape=["N", 9])            # bytes of a ModelProto
    open("model.onnx", "wb").write(data)

Layers: Linear (Gemm, or MatMul + Add on inputs of rank > 2), Embedding (Gather), LayerNorm (LayerNormalization),
RMSNorm (Mul / ReduceMean / Sqrt / Div), PositionalEncoding (Slice-free Add on a fixed length), MultiHeadAttention and
TransformerEncoderLayer (MatMul, Reshape, Transpose, Softmax, causal mask as a constant), Conv1d / Conv2d /
ConvTranspose2d, BatchNorm2d (inference form), GroupNorm (InstanceNormalization on regrouped channels), pools,
Upsample (Resize), Flatten, Dropout (dropped), activations.

Reference: the reference's exporter and graph writer (src/Idrak/Onnx/OnnxExport.cs, OnnxGraphWriter.cs).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch
from torch import nn

from ..nn import layers as L
from . import proto as P


class GraphWriter:
    def __init__(self, name: str = "network"):
        self.graph = P.Graph(name)
        self._n = 0

    def fresh(self, hint: str = "v") -> str:
        self._n += 1
        return f"{hint}_{self._n}"

    def const(self, value, hint: str = "c") -> str:
        name = self.fresh(hint)
        t = value.detach().cpu().float().numpy() if isinstance(value, torch.Tensor) and value.is_floating_point() else \
            (value.detach().cpu().numpy() if isinstance(value, torch.Tensor) else np.asarray(value))
        self.graph.initializers[name] = t
        return name

    def ints(self, values: Sequence[int]) -> str:
        return self.const(np.asarray(values, np.int64), "shape")

    def node(self, op: str, inputs: Sequence[str], outputs: int = 1, **attributes) -> Union[str, List[str]]:
        outs = [self.fresh(op.lower()) for _ in range(outputs)]
        self.graph.nodes.append(P.Node(op, list(inputs), outs, {k: v for k, v in attributes.items() if v is not None},
                                       name=f"{op}_{len(self.graph.nodes)}"))
        return outs[0] if outputs == 1 else outs


def _linear(w: GraphWriter, m, x: str, rank: int) -> str:
    if rank == 2:
        ins = [x, w.const(m.weight, "weight")] + ([w.const(m.bias, "bias")] if m.bias is not None else [])
        return w.node("Gemm", ins, transB=1)
    y = w.node("MatMul", [x, w.const(m.weight.detach().t().contiguous(), "weight")])
    return w.node("Add", [y, w.const(m.bias, "bias")]) if m.bias is not None else y


def _attention(w: GraphWriter, m: L.MultiHeadAttention, x: str, length: int) -> str:
    H, D = m.heads, m.dim // m.heads
    qkv = _linear(w, m.qkv, x, 3)                                               # [N, T, 3 C]
    qkv = w.node("Reshape", [qkv, w.ints([0, 0, 3, H, D])])
    qkv = w.node("Transpose", [qkv], perm=[2, 0, 3, 1, 4])                       # [3, N, H, T, D]
    q, k, v = w.node("Split", [qkv, w.ints([1, 1, 1])], outputs=3, axis=0)
    q, k, v = (w.node("Squeeze", [t, w.ints([0])]) for t in (q, k, v))
    s = w.node("MatMul", [q, w.node("Transpose", [k], perm=[0, 1, 3, 2])])
    s = w.node("Mul", [s, w.const(np.float32(1.0 / math.sqrt(D)), "scale")])
    if m.causal:
        mask = np.triu(np.full((length, length), -1e30, np.float32), 1)
        s = w.node("Add", [s, w.const(mask, "causal")])
    a = w.node("MatMul", [w.node("Softmax", [s], axis=-1), v])                   # [N, H, T, D]
    a = w.node("Reshape", [w.node("Transpose", [a], perm=[0, 2, 1, 3]), w.ints([0, 0, H * D])])
    return _linear(w, m.out, a, 3)


def _layer_norm(w: GraphWriter, m, x: str) -> str:
    return w.node("LayerNormalization", [x, w.const(m.weight, "gamma"), w.const(m.bias, "beta")], axis=-1,
                  epsilon=float(getattr(m, "epsilon", getattr(m, "eps", 1e-5))))


def _pair(v):
    return list(v) if isinstance(v, (tuple, list)) else [v, v]


def _add_layer(w: GraphWriter, m: nn.Module, x: str, shape: List) -> str:
    """Append ``m`` applied to value ``x`` whose sample shape (without the batch dimension) is ``shape``."""
    rank = len(shape) + 1
    if isinstance(m, (L.Linear, nn.Linear)):
        return _linear(w, m, x, rank)
    if isinstance(m, (L.Embedding, nn.Embedding)):
        return w.node("Gather", [w.const(m.weight, "table"), x], axis=0)
    if isinstance(m, (L.LayerNorm, nn.LayerNorm)):
        return _layer_norm(w, m, x)
    if isinstance(m, L.RMSNorm):
        ms = w.node("ReduceMean", [w.node("Mul", [x, x])], axes=[-1], keepdims=1)
        rms = w.node("Sqrt", [w.node("Add", [ms, w.const(np.float32(m.epsilon), "eps")])])
        return w.node("Mul", [w.node("Div", [x, rms]), w.const(m.weight, "gamma")])
    if isinstance(m, L.PositionalEncoding):
        return w.node("Add", [x, w.const(m.table[: shape[0]], "positions")])
    if isinstance(m, L.MultiHeadAttention):
        return _attention(w, m, x, shape[0])
    if isinstance(m, L.TransformerEncoderLayer):
        act = "Gelu" if m.activation == "gelu" else "Relu"

        def ff(h):
            u = _linear(w, m.up, h, 3)
            u = _gelu(w, u, False) if act == "Gelu" else w.node("Relu", [u])
            return _linear(w, m.down, u, 3)
        if m.norms == "before":
            x = w.node("Add", [x, _attention(w, m.attention, _layer_norm(w, m.norm1, x), shape[0])])
            return w.node("Add", [x, ff(_layer_norm(w, m.norm2, x))])
        x = _layer_norm(w, m.norm1, w.node("Add", [x, _attention(w, m.attention, x, shape[0])]))
        return _layer_norm(w, m.norm2, w.node("Add", [x, ff(x)]))
    if isinstance(m, (nn.Conv1d, nn.Conv2d)):
        ins = [x, w.const(m.weight, "kernel")] + ([w.const(m.bias, "bias")] if m.bias is not None else [])
        pads = list(m.padding) * 2
        return w.node("Conv", ins, kernel_shape=list(m.kernel_size), strides=list(m.stride), pads=pads,
                      dilations=list(m.dilation), group=m.groups)
    if isinstance(m, nn.ConvTranspose2d):
        ins = [x, w.const(m.weight, "kernel")] + ([w.const(m.bias, "bias")] if m.bias is not None else [])
        return w.node("ConvTranspose", ins, kernel_shape=list(m.kernel_size), strides=list(m.stride), pads=list(m.padding) * 2,
                      output_padding=list(m.output_padding), dilations=list(m.dilation), group=m.groups)
    if isinstance(m, nn.BatchNorm2d):
        return w.node("BatchNormalization", [x, w.const(m.weight, "gamma"), w.const(m.bias, "beta"),
                                             w.const(m.running_mean, "mean"), w.const(m.running_var, "var")], epsilon=float(m.eps))
    if isinstance(m, nn.GroupNorm):
        C, G = m.num_channels, m.num_groups
        g = w.node("Reshape", [x, w.ints([0, G, -1])])
        g = w.node("InstanceNormalization", [g, w.const(np.ones(G, np.float32)), w.const(np.zeros(G, np.float32))], epsilon=float(m.eps))
        y = w.node("Reshape", [g, w.node("Shape", [x])])
        if m.affine:
            view = [C] + [1] * (len(shape) - 1)
            y = w.node("Add", [w.node("Mul", [y, w.const(m.weight.detach().view(view), "gamma")]), w.const(m.bias.detach().view(view), "beta")])
        return y
    if isinstance(m, nn.MaxPool2d):
        return w.node("MaxPool", [x], kernel_shape=_pair(m.kernel_size), strides=_pair(m.stride), pads=_pair(m.padding) * 2,
                      ceil_mode=int(m.ceil_mode))
    if isinstance(m, nn.AvgPool2d):
        return w.node("AveragePool", [x], kernel_shape=_pair(m.kernel_size), strides=_pair(m.stride), pads=_pair(m.padding) * 2,
                      ceil_mode=int(m.ceil_mode), count_include_pad=int(m.count_include_pad))
    if isinstance(m, L.GlobalAveragePool2d):
        return w.node("Flatten", [w.node("GlobalAveragePool", [x])], axis=1)
    if isinstance(m, nn.AdaptiveAvgPool2d):
        out = _pair(m.output_size)
        H, Wd = shape[1], shape[2]
        if H % out[0] or Wd % out[1]:
            raise ValueError("adaptive pooling exports only when the output size divides the input size")
        k = [H // out[0], Wd // out[1]]
        return w.node("AveragePool", [x], kernel_shape=k, strides=k)
    if isinstance(m, nn.Upsample):
        mode = {"nearest": "nearest", "bilinear": "linear"}[m.mode]
        kw = dict(mode=mode, coordinate_transformation_mode="asymmetric" if mode == "nearest" else
                  ("align_corners" if m.align_corners else "half_pixel"))
        if mode == "nearest":
            kw["nearest_mode"] = "floor"
        if m.size is not None:
            sizes = w.node("Concat", [w.node("Slice", [w.node("Shape", [x]), w.ints([0]), w.ints([2])]), w.ints(_pair(m.size))], axis=0)
            return w.node("Resize", [x, "", "", sizes], **kw)
        sf = m.scale_factor if isinstance(m.scale_factor, (tuple, list)) else (m.scale_factor, m.scale_factor)
        return w.node("Resize", [x, "", w.const(np.asarray([1.0, 1.0, *sf], np.float32), "scales")], **kw)
    if isinstance(m, nn.Flatten):
        return w.node("Flatten", [x], axis=1)
    if isinstance(m, (nn.Dropout, nn.Identity)):
        return x
    if isinstance(m, nn.GELU):
        return _gelu(w, x, m.approximate == "tanh")
    if isinstance(m, L.QuickGELU):
        return w.node("Mul", [x, w.node("Sigmoid", [w.node("Mul", [x, w.const(np.float32(1.702))])])])
    if isinstance(m, nn.Softmax):
        return w.node("Softmax", [x], axis=-1)
    for cls, op in ((nn.ReLU, "Relu"), (nn.Tanh, "Tanh"), (nn.Sigmoid, "Sigmoid")):
        if isinstance(m, cls):
            return w.node(op, [x])
    if isinstance(m, nn.Sequential):
        for child in m:
            x, shape = _add_tracked(w, child, x, shape)
        return x
    raise NotImplementedError(f"{type(m).__name__} has no ONNX export here")


def _gelu(w: GraphWriter, x: str, tanh: bool) -> str:
    """GELU from opset-17 operators (the Gelu operator itself arrives in opset 20)."""
    if tanh:
        x3 = w.node("Mul", [w.node("Mul", [x, x]), x])
        inner = w.node("Mul", [w.node("Add", [x, w.node("Mul", [x3, w.const(np.float32(0.044715))])]),
                               w.const(np.float32(math.sqrt(2.0 / math.pi)))])
        return w.node("Mul", [w.node("Mul", [x, w.const(np.float32(0.5))]), w.node("Add", [w.node("Tanh", [inner]), w.const(np.float32(1.0))])])
    erf = w.node("Erf", [w.node("Mul", [x, w.const(np.float32(1.0 / math.sqrt(2.0)))])])
    return w.node("Mul", [w.node("Mul", [x, w.const(np.float32(0.5))]), w.node("Add", [erf, w.const(np.float32(1.0))])])


def _add_tracked(w, m, x, shape):
    y = _add_layer(w, m, x, shape)
    was = m.training
    m.eval()
    with torch.no_grad():
        ids = isinstance(m, (L.Embedding, nn.Embedding))
        probe = torch.zeros(1, *shape, dtype=torch.long if ids else torch.float32)
        out = m(probe)
    m.train(was)
    return y, list(out.shape[1:])


def export(model: nn.Module, input_shape: Sequence[Union[int, str]], input_name: str = "input", output_name: str = "output",
           integer_input: bool = False) -> bytes:
    """``input_shape`` includes the batch dimension, which may be a name (``["N", 9]``); the other sizes are fixed."""
    w = GraphWriter(type(model).__name__)
    sample = [int(v) for v in input_shape[1:]]
    layers = list(model) if isinstance(model, nn.Sequential) else [model]
    first_ids = integer_input or (layers and isinstance(layers[0], (L.Embedding, nn.Embedding)))
    w.graph.inputs.append(P.ValueInfo(input_name, P.INT64 if first_ids else P.FLOAT, list(input_shape)))
    x, shape = input_name, sample
    params = [p for p in model.parameters()]
    model_cpu = model if not params or not params[0].is_cuda else None
    if model_cpu is None:
        raise ValueError("export a model that lives on the CPU (model.cpu().float())")
    for m in layers:
        x, shape = _add_tracked(w, m, x, shape)
    w.graph.nodes.append(P.Node("Identity", [x], [output_name], name="output"))
    w.graph.outputs.append(P.ValueInfo(output_name, P.FLOAT, [input_shape[0]] + shape))
    return P.Model(w.graph, opset=17).serialize()
