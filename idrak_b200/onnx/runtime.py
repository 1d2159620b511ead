"""Run ONNX graphs with tensor ops: ``OnnxModule(bytes)`` is an ``nn.Module`` whose initialisers are parameters /
buffers and whose ``forward`` walks the graph in order. Covers the operators PyTorch's exporter emits for dense,
convolutional, recurrent and attention models (about sixty); an operator outside the table raises by name.

    module = load("model.onnx")
    y = module(x)                       # one output -> a tensor, several -> a tuple

Reference: the reference's importer (src/Idrak/Onnx/OnnxImport.cs, OnnxBuiltIns.cs: operator table, shape
arithmetic on small integer tensors, LSTM / GRU with ONNX's gate order).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from . import proto as P

TORCH_TYPES = {P.FLOAT: torch.float32, P.UINT8: torch.uint8, P.INT8: torch.int8, P.INT16: torch.int16, P.INT32: torch.int32,
               P.INT64: torch.int64, P.BOOL: torch.bool, P.FLOAT16: torch.float16, P.DOUBLE: torch.float64,
               P.BFLOAT16: torch.bfloat16}
OPS: Dict[str, Callable] = {}


def op(*names):
    def add(fn):
        for n in names:
            OPS[n] = fn
        return fn
    return add


def _ints(t) -> List[int]:
    return [int(v) for v in (t.tolist() if isinstance(t, torch.Tensor) else t)]


def _pads(attrs, dims: int) -> List[int]:
    """ONNX pads (begin..., end...) -> F.pad order (last dim first, begin / end pairs)."""
    p = attrs.get("pads") or [0] * (2 * dims)
    out = []
    for d in reversed(range(dims)):
        out += [p[d], p[d + dims]]
    return out


def _auto_pad(attrs, x, kernel, strides, dilations) -> List[int]:
    mode = attrs.get("auto_pad", "NOTSET")
    dims = len(kernel)
    if mode in ("NOTSET", "", "VALID"):
        return _pads(attrs, dims) if mode != "VALID" else [0] * (2 * dims)
    out = []
    for d in reversed(range(dims)):
        size = x.shape[2 + d]
        total = max((math.ceil(size / strides[d]) - 1) * strides[d] + (kernel[d] - 1) * dilations[d] + 1 - size, 0)
        lo = total // 2 if mode == "SAME_UPPER" else total - total // 2
        out += [lo, total - lo]
    return out


# ------------------------------------------------------------------------------------------------ element-wise / math
for _name, _fn in (("Relu", torch.relu), ("Tanh", torch.tanh), ("Sigmoid", torch.sigmoid), ("Exp", torch.exp), ("Log", torch.log),
                   ("Sqrt", torch.sqrt), ("Erf", torch.erf), ("Abs", torch.abs), ("Neg", torch.neg), ("Floor", torch.floor),
                   ("Ceil", torch.ceil), ("Reciprocal", torch.reciprocal), ("Sin", torch.sin), ("Cos", torch.cos),
                   ("Not", torch.logical_not), ("Softplus", F.softplus), ("Identity", lambda x: x), ("Sign", torch.sign)):
    OPS[_name] = (lambda f: lambda a, x: f(x))(_fn)
for _name, _fn in (("Add", torch.add), ("Sub", torch.sub), ("Mul", torch.mul), ("Pow", torch.pow), ("Equal", torch.eq),
                   ("Less", torch.lt), ("Greater", torch.gt), ("And", torch.logical_and), ("Or", torch.logical_or),
                   ("Max", torch.maximum), ("Min", torch.minimum), ("MatMul", torch.matmul)):
    OPS[_name] = (lambda f: lambda a, x, y: f(x, y))(_fn)


@op("Div")
def _div(a, x, y):
    if not x.is_floating_point() and not y.is_floating_point():
        return torch.div(x, y, rounding_mode="trunc")
    return x / y


@op("Gelu")
def _gelu(a, x):
    return F.gelu(x, approximate="tanh" if a.get("approximate") == "tanh" else "none")


@op("LeakyRelu")
def _leaky(a, x):
    return F.leaky_relu(x, a.get("alpha", 0.01))


@op("Elu")
def _elu(a, x):
    return F.elu(x, a.get("alpha", 1.0))


@op("HardSigmoid")
def _hard_sigmoid(a, x):
    return (x * a.get("alpha", 0.2) + a.get("beta", 0.5)).clamp(0, 1)


@op("HardSwish")
def _hard_swish(a, x):
    return F.hardswish(x)


@op("Clip")
def _clip(a, x, lo=None, hi=None):
    lo = a.get("min") if lo is None else lo
    hi = a.get("max") if hi is None else hi
    return x.clamp(min=None if lo is None else float(lo), max=None if hi is None else float(hi))


@op("Softmax")
def _softmax(a, x):
    return F.softmax(x, a.get("axis", -1))


@op("LogSoftmax")
def _log_softmax(a, x):
    return F.log_softmax(x, a.get("axis", -1))


@op("Where")
def _where(a, c, x, y):
    return torch.where(c.bool(), x, y)


@op("Cast")
def _cast(a, x):
    return x.to(TORCH_TYPES[a["to"]])


@op("Dropout")
def _dropout(a, x, *rest):
    return x


@op("Gemm")
def _gemm(a, x, w, b=None):
    x = x.t() if a.get("transA", 0) else x
    w = w.t() if a.get("transB", 0) else w
    y = a.get("alpha", 1.0) * (x @ w)
    return y if b is None else y + a.get("beta", 1.0) * b


# ------------------------------------------------------------------------------------------------ reductions
def _reduce(fn):
    def run(a, x, axes=None):
        ax = _ints(axes) if axes is not None else a.get("axes")
        keep = bool(a.get("keepdims", 1))
        if not ax:
            if a.get("noop_with_empty_axes", 0):
                return x
            ax = list(range(x.dim()))
        return fn(x, ax, keep)
    return run


OPS["ReduceMean"] = _reduce(lambda x, ax, k: x.mean(ax, keepdim=k))
OPS["ReduceSum"] = _reduce(lambda x, ax, k: x.sum(ax, keepdim=k))
OPS["ReduceMax"] = _reduce(lambda x, ax, k: x.amax(ax, keepdim=k))
OPS["ReduceMin"] = _reduce(lambda x, ax, k: x.amin(ax, keepdim=k))
OPS["ReduceL2"] = _reduce(lambda x, ax, k: x.pow(2).sum(ax, keepdim=k).sqrt())


@op("ArgMax")
def _argmax(a, x):
    return x.argmax(a.get("axis", 0), keepdim=bool(a.get("keepdims", 1)))


# ------------------------------------------------------------------------------------------------ shapes
@op("Shape")
def _shape(a, x):
    s = list(x.shape)[a.get("start", 0): a.get("end")]
    return torch.tensor(s, dtype=torch.int64)


@op("Reshape")
def _reshape(a, x, shape):
    s = _ints(shape)
    s = [x.shape[i] if (v == 0 and not a.get("allowzero", 0)) else v for i, v in enumerate(s)]
    return x.reshape(s)


@op("Flatten")
def _flatten(a, x):
    ax = a.get("axis", 1)
    return x.reshape(int(np.prod(x.shape[:ax])) if ax else 1, -1)


@op("Transpose")
def _transpose(a, x):
    return x.permute(a.get("perm") or list(reversed(range(x.dim()))))


@op("Squeeze")
def _squeeze(a, x, axes=None):
    ax = _ints(axes) if axes is not None else a.get("axes")
    if not ax:
        return x.squeeze()
    for d in sorted((d % x.dim() for d in ax), reverse=True):
        x = x.squeeze(d)
    return x


@op("Unsqueeze")
def _unsqueeze(a, x, axes=None):
    ax = _ints(axes) if axes is not None else a["axes"]
    rank = x.dim() + len(ax)
    for d in sorted(d % rank for d in ax):
        x = x.unsqueeze(d)
    return x


@op("Concat")
def _concat(a, *xs):
    return torch.cat([x for x in xs if x.numel() or x.dim() > 1], a["axis"])


@op("Split")
def _split(a, x, split=None):
    ax = a.get("axis", 0)
    sizes = _ints(split) if split is not None else a.get("split")
    if sizes is None:
        n = a.get("num_outputs", 2)
        sizes = math.ceil(x.shape[ax] / n)
    return tuple(torch.split(x, sizes, ax))


@op("Slice")
def _slice(a, x, starts=None, ends=None, axes=None, steps=None):
    starts = _ints(starts) if starts is not None else a["starts"]
    ends = _ints(ends) if ends is not None else a["ends"]
    axes = _ints(axes) if axes is not None else a.get("axes") or list(range(len(starts)))
    steps = _ints(steps) if steps is not None else [1] * len(starts)
    for s, e, ax, st in zip(starts, ends, axes, steps):
        n = x.shape[ax]
        s = s + n if s < 0 else s
        e = e + n if e < 0 else e
        if st > 0:
            s, e = min(max(s, 0), n), min(max(e, 0), n)
        else:
            s, e = min(max(s, 0), n - 1), min(max(e, -1), n - 1)     # an end below -n means "through element 0"
        x = x.index_select(ax, torch.arange(s, e, st, device=x.device))
    return x


@op("Gather")
def _gather(a, x, idx):
    ax = a.get("axis", 0)
    i = idx.long()
    i = torch.where(i < 0, i + x.shape[ax], i)
    if i.dim() == 0:
        return x.select(ax, int(i))
    return x.index_select(ax, i.reshape(-1)).reshape(*x.shape[:ax], *i.shape, *x.shape[ax + 1:] if ax != -1 else ())


@op("Expand")
def _expand(a, x, shape):
    s = _ints(shape)
    return x * torch.ones(s, dtype=x.dtype, device=x.device) if x.dtype != torch.bool else x.expand(torch.broadcast_shapes(x.shape, s))


@op("Tile")
def _tile(a, x, reps):
    return x.repeat(_ints(reps))


@op("ConstantOfShape")
def _constant_of_shape(a, shape):
    v = a.get("value")
    fill = torch.from_numpy(np.array(v.array)).reshape(-1)[0] if v is not None else torch.tensor(0.0)
    return torch.full(_ints(shape), fill.item(), dtype=fill.dtype)


@op("Range")
def _range(a, start, limit, delta):
    return torch.arange(start.item(), limit.item(), delta.item(), dtype=start.dtype)


@op("Constant")
def _constant(a):
    if "value" in a:
        return torch.from_numpy(np.array(a["value"].array))
    for k, dt in (("value_float", torch.float32), ("value_int", torch.int64), ("value_floats", torch.float32), ("value_ints", torch.int64)):
        if k in a:
            return torch.tensor(a[k], dtype=dt)
    raise P.ProtoError("Constant without a value")


@op("Pad")
def _pad(a, x, pads=None, value=None, axes=None):
    p = _ints(pads) if pads is not None else a["pads"]
    dims = len(p) // 2
    ax = _ints(axes) if axes is not None else list(range(dims))
    full = [0] * (2 * x.dim())
    for j, d in enumerate(ax):
        full[d], full[d + x.dim()] = p[j], p[j + dims]
    tp = []
    for d in reversed(range(x.dim())):
        tp += [full[d], full[d + x.dim()]]
    mode = {"constant": "constant", "reflect": "reflect", "edge": "replicate"}[a.get("mode", "constant")]
    fill = float(value) if value is not None and value.numel() else float(a.get("value", 0.0))
    return F.pad(x, tp, mode=mode, value=fill) if mode == "constant" else F.pad(x, tp, mode=mode)


# ------------------------------------------------------------------------------------------------ layers
@op("Conv")
def _conv(a, x, w, b=None):
    dims = w.dim() - 2
    strides = a.get("strides") or [1] * dims
    dil = a.get("dilations") or [1] * dims
    pads = _auto_pad(a, x, list(w.shape[2:]), strides, dil)
    if any(pads):
        x = F.pad(x, pads)
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[dims]
    return fn(x, w, b, strides, 0, dil, a.get("group", 1))


@op("ConvTranspose")
def _conv_transpose(a, x, w, b=None):
    dims = w.dim() - 2
    p = a.get("pads") or [0] * (2 * dims)
    if p[:dims] != p[dims:]:
        raise P.ProtoError("ConvTranspose with uneven padding is not run")
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d}[dims]
    return fn(x, w, b, a.get("strides") or [1] * dims, p[:dims], a.get("output_padding") or [0] * dims, a.get("group", 1),
              a.get("dilations") or [1] * dims)


def _pool(kind):
    def run(a, x):
        k = a["kernel_shape"]
        dims = len(k)
        strides = a.get("strides") or [1] * dims
        dil = a.get("dilations") or [1] * dims
        pads = _auto_pad(a, x, k, strides, dil)
        ceil = bool(a.get("ceil_mode", 0))
        sym = all(pads[2 * i] == pads[2 * i + 1] for i in range(dims))
        pad = [pads[2 * i] for i in reversed(range(dims))]
        if kind == "max":
            if not sym:
                x, pad = F.pad(x, pads, value=float("-inf")), [0] * dims
            return {1: F.max_pool1d, 2: F.max_pool2d}[dims](x, k, strides, pad, dil, ceil)
        include = bool(a.get("count_include_pad", 0))
        if not sym:
            if not include:
                raise P.ProtoError("AveragePool with uneven padding that is not counted is not run")
            x, pad = F.pad(x, pads), [0] * dims
        return {1: F.avg_pool1d, 2: F.avg_pool2d}[dims](x, k, strides, pad, ceil, include)
    return run


OPS["MaxPool"] = _pool("max")
OPS["AveragePool"] = _pool("avg")


@op("GlobalAveragePool")
def _gap(a, x):
    return x.mean(tuple(range(2, x.dim())), keepdim=True)


@op("GlobalMaxPool")
def _gmp(a, x):
    return x.amax(tuple(range(2, x.dim())), keepdim=True)


@op("BatchNormalization")
def _bn(a, x, scale, bias, mean, var):
    return F.batch_norm(x, mean, var, scale, bias, False, 0.0, a.get("epsilon", 1e-5))


@op("InstanceNormalization")
def _in(a, x, scale, bias):
    return F.instance_norm(x, weight=scale, bias=bias, eps=a.get("epsilon", 1e-5))


@op("LayerNormalization")
def _ln(a, x, scale, bias=None):
    ax = a.get("axis", -1) % x.dim()
    return F.layer_norm(x, x.shape[ax:], scale, bias, a.get("epsilon", 1e-5))


@op("Resize", "Upsample")
def _resize(a, x, roi=None, scales=None, sizes=None):
    mode = a.get("mode", "nearest")
    if sizes is not None and sizes.numel():
        size, factor = _ints(sizes)[2:], None
    else:
        s = scales if scales is not None and scales.numel() else roi
        size, factor = None, [float(v) for v in s.tolist()[2:]]
    if mode == "nearest":
        return F.interpolate(x, size=size, scale_factor=factor, mode="nearest")
    align = a.get("coordinate_transformation_mode", "half_pixel") == "align_corners"
    return F.interpolate(x, size=size, scale_factor=factor, mode={"linear": "bilinear", "cubic": "bicubic"}[mode], align_corners=align)


def _act(name: str):
    return {"Sigmoid": torch.sigmoid, "Tanh": torch.tanh, "Relu": torch.relu}[name]


@op("LSTM")
def _lstm(a, x, w, r, b=None, seq_lens=None, h0=None, c0=None, p=None):
    """X [T, N, I] (or [N, T, I] with layout 1); W [dirs, 4H, I] and R [dirs, 4H, H] in gate order i, o, f, c."""
    if a.get("layout", 0):
        x = x.transpose(0, 1)
    T, N, _ = x.shape
    H = a["hidden_size"]
    dirs = w.shape[0]
    ys, hs, cs = [], [], []
    for d in range(dirs):
        reverse = (a.get("direction", "forward") == "reverse") or d == 1
        bias = (b[d, : 4 * H] + b[d, 4 * H:]) if b is not None else 0
        h = h0[d] if h0 is not None else x.new_zeros(N, H)
        c = c0[d] if c0 is not None else x.new_zeros(N, H)
        out = [None] * T
        for t in (range(T - 1, -1, -1) if reverse else range(T)):
            g = x[t] @ w[d].t() + h @ r[d].t() + bias
            i, o, f, cc = g.split(H, -1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(cc)
            h = torch.sigmoid(o) * torch.tanh(c)
            out[t] = h
        ys.append(torch.stack(out))
        hs.append(h)
        cs.append(c)
    y = torch.stack(ys, 1)                                   # [T, dirs, N, H]
    if a.get("layout", 0):
        y = y.permute(2, 0, 1, 3)
    return y, torch.stack(hs), torch.stack(cs)


@op("GRU")
def _gru(a, x, w, r, b=None, seq_lens=None, h0=None):
    """Gate order z, r, h. ``linear_before_reset`` 1 is PyTorch's form."""
    if a.get("layout", 0):
        x = x.transpose(0, 1)
    T, N, _ = x.shape
    H = a["hidden_size"]
    lbr = a.get("linear_before_reset", 0)
    ys, hs = [], []
    for d in range(w.shape[0]):
        reverse = (a.get("direction", "forward") == "reverse") or d == 1
        wb = b[d, : 3 * H] if b is not None else x.new_zeros(3 * H)
        rb = b[d, 3 * H:] if b is not None else x.new_zeros(3 * H)
        h = h0[d] if h0 is not None else x.new_zeros(N, H)
        out = [None] * T
        for t in (range(T - 1, -1, -1) if reverse else range(T)):
            gx = x[t] @ w[d].t() + wb
            xz, xr, xh = gx.split(H, -1)
            rz, rr, rh = r[d].split(H, 0)
            z = torch.sigmoid(xz + h @ rz.t() + rb[:H])
            rg = torch.sigmoid(xr + h @ rr.t() + rb[H: 2 * H])
            if lbr:
                cand = torch.tanh(xh + rg * (h @ rh.t() + rb[2 * H:]))
            else:
                cand = torch.tanh(xh + (rg * h) @ rh.t() + rb[2 * H:])
            h = (1 - z) * cand + z * h
            out[t] = h
        ys.append(torch.stack(out))
        hs.append(h)
    y = torch.stack(ys, 1)
    if a.get("layout", 0):
        y = y.permute(2, 0, 1, 3)
    return y, torch.stack(hs)


# ---------------------------------------------------------------------------------------------------------------------
class OnnxModule(nn.Module):
    def __init__(self, model: P.Model, trainable: bool = False):
        super().__init__()
        self.model = model
        g = model.graph
        missing = sorted({n.op_type for n in g.nodes if n.op_type not in OPS})
        if missing:
            raise NotImplementedError(f"ONNX operators not run here: {', '.join(missing)} (opset {model.opset})")
        self._names: Dict[str, str] = {}
        for i, (name, arr) in enumerate(g.initializers.items()):
            t = torch.from_numpy(np.array(arr))
            key = f"t{i}"
            self._names[name] = key
            if trainable and t.is_floating_point():
                self.register_parameter(key, nn.Parameter(t))
            else:
                self.register_buffer(key, t)
        self.input_names = [vi.name for vi in g.inputs if vi.name not in g.initializers]
        self.output_names = [vi.name for vi in g.outputs]

    def forward(self, *inputs, **named):
        g = self.model.graph
        env: Dict[str, Optional[torch.Tensor]] = {"": None}
        for name, key in self._names.items():
            env[name] = getattr(self, key)
        if len(inputs) > len(self.input_names):
            raise ValueError(f"the graph takes {len(self.input_names)} inputs: {', '.join(self.input_names)}")
        for name, value in list(zip(self.input_names, inputs)) + list(named.items()):
            if name not in self.input_names:
                raise KeyError(f"no graph input '{name}'; inputs: {', '.join(self.input_names)}")
            env[name] = value
        dev = next((v.device for v in env.values() if isinstance(v, torch.Tensor) and v.is_cuda), None)
        for node in g.nodes:
            args = [env[i] for i in node.inputs]
            while args and args[-1] is None:
                args.pop()
            out = OPS[node.op_type](node.attributes, *args)
            outs = out if isinstance(out, tuple) else (out,)
            for name, value in zip(node.outputs, outs):
                if name:
                    if dev is not None and isinstance(value, torch.Tensor) and not value.is_cuda and value.is_floating_point():
                        value = value.to(dev)
                    env[name] = value
        res = tuple(env[n] for n in self.output_names)
        return res[0] if len(res) == 1 else res


def load(source, trainable: bool = False) -> OnnxModule:
    """An ONNX file (path or bytes) as a module."""
    data = source if isinstance(source, (bytes, bytearray)) else open(source, "rb").read()
    return OnnxModule(P.Model.parse(bytes(data)), trainable)
