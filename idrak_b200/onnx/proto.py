"""The slice of protocol buffers that ONNX files need, written out by hand: varints, length-delimited fields, and the
ONNX messages (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto, ValueInfoProto) as small Python
classes with ``parse`` / ``serialize``. No ``protobuf`` or ``onnx`` package is used.

Field numbers follow onnx.proto3 (ModelProto: ir_version 1, producer_name 2, graph 7, opset_import 8; GraphProto: node 1,
name 2, initializer 5, input 11, output 12, value_info 13; NodeProto: input 1, output 2, name 3, op_type 4,
attribute 5, domain 7; AttributeProto: name 1, f 2, i 3, s 4, t 5, g 6, floats 7, ints 8, strings 9, type 20;
TensorProto: dims 1, data_type 2, float_data 4, int32_data 5, int64_data 7, name 8, raw_data 9, double_data 10).

Reference: the reference's own protobuf reader / writer (src/Idrak/Onnx/Protobuf.cs) and model classes (OnnxModel.cs).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Tuple, Union

import numpy as np

# TensorProto.DataType
FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL, FLOAT16, DOUBLE, UINT32, UINT64, BFLOAT16 = \
    1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 16
NUMPY_TYPES = {FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, UINT16: np.uint16, INT16: np.int16, INT32: np.int32,
               INT64: np.int64, BOOL: np.bool_, FLOAT16: np.float16, DOUBLE: np.float64, UINT32: np.uint32, UINT64: np.uint64}
ONNX_TYPES = {np.dtype(v): k for k, v in NUMPY_TYPES.items()}
# AttributeProto.AttributeType
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_GRAPH, A_FLOATS, A_INTS, A_STRINGS = 1, 2, 3, 4, 5, 6, 7, 8


class ProtoError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------------------------------
# wire format
# ---------------------------------------------------------------------------------------------------------------------
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, at: int) -> Tuple[int, int]:
    v = shift = 0
    while True:
        if at >= len(buf):
            raise ProtoError("truncated varint")
        b = buf[at]
        at += 1
        v |= (b & 0x7F) << shift
        if not b & 0x80:
            return v, at
        shift += 7
        if shift > 70:
            raise ProtoError("varint too long")


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def fields(buf: bytes) -> Iterator[Tuple[int, int, Union[int, bytes]]]:
    """(field number, wire type, value) for every field of a message."""
    at = 0
    while at < len(buf):
        key, at = _read_varint(buf, at)
        num, wire = key >> 3, key & 7
        if wire == 0:
            v, at = _read_varint(buf, at)
            yield num, wire, v
        elif wire == 1:
            yield num, wire, buf[at: at + 8]
            at += 8
        elif wire == 2:
            n, at = _read_varint(buf, at)
            if at + n > len(buf):
                raise ProtoError("truncated field")
            yield num, wire, buf[at: at + n]
            at += n
        elif wire == 5:
            yield num, wire, buf[at: at + 4]
            at += 4
        else:
            raise ProtoError(f"wire type {wire} is not read")


class Writer:
    def __init__(self):
        self.parts: List[bytes] = []

    def varint(self, num: int, v: int) -> None:
        self.parts.append(_varint(num << 3) + _varint(int(v)))

    def bytes(self, num: int, v: bytes) -> None:
        self.parts.append(_varint(num << 3 | 2) + _varint(len(v)) + v)

    def string(self, num: int, v: str) -> None:
        self.bytes(num, v.encode("utf-8"))

    def float32(self, num: int, v: float) -> None:
        self.parts.append(_varint(num << 3 | 5) + struct.pack("<f", v))

    def packed_varints(self, num: int, vs) -> None:
        self.bytes(num, b"".join(_varint(int(v)) for v in vs))

    def packed_floats(self, num: int, vs) -> None:
        self.bytes(num, struct.pack(f"<{len(vs)}f", *vs))

    def done(self) -> bytes:
        return b"".join(self.parts)


def _packed_ints(wire: int, v) -> List[int]:
    if wire == 0:
        return [_signed(v)]
    out, at = [], 0
    while at < len(v):
        x, at = _read_varint(v, at)
        out.append(_signed(x))
    return out


def _packed_floats(wire: int, v, fmt: str = "<f") -> List[float]:
    size = struct.calcsize(fmt)
    return [struct.unpack(fmt, v[i: i + size])[0] for i in range(0, len(v), size)]


# ---------------------------------------------------------------------------------------------------------------------
# messages
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Tensor:
    name: str = ""
    array: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))

    @classmethod
    def parse(cls, buf: bytes) -> "Tensor":
        dims: List[int] = []
        dtype, name, raw = FLOAT, "", None
        floats: List[float] = []
        ints: List[int] = []
        doubles: List[float] = []
        for num, wire, v in fields(buf):
            if num == 1:
                dims += _packed_ints(wire, v)
            elif num == 2:
                dtype = v
            elif num == 4:
                floats += _packed_floats(wire, v)
            elif num in (5, 7, 11):
                ints += _packed_ints(wire, v)
            elif num == 8:
                name = v.decode("utf-8")
            elif num == 9:
                raw = v
            elif num == 10:
                doubles += _packed_floats(wire, v, "<d")
            elif num == 13 and v:
                raise ProtoError(f"tensor '{name}' keeps its data in an external file, which is not read")
        if dtype == BFLOAT16:
            words = np.frombuffer(raw, "<u2") if raw is not None else np.asarray(ints, np.uint16)
            arr = (words.astype(np.uint32) << 16).view(np.float32)
        elif dtype not in NUMPY_TYPES:
            raise ProtoError(f"tensor '{name}': data type {dtype} is not read")
        elif raw is not None:
            arr = np.frombuffer(raw, np.dtype(NUMPY_TYPES[dtype]).newbyteorder("<")).astype(NUMPY_TYPES[dtype])
        elif dtype == FLOAT:
            arr = np.asarray(floats, np.float32)
        elif dtype == DOUBLE:
            arr = np.asarray(doubles, np.float64)
        elif dtype == FLOAT16:
            arr = np.asarray(ints, np.uint16).view(np.float16)
        else:
            arr = np.asarray(ints).astype(NUMPY_TYPES[dtype])
        return cls(name, arr.reshape(dims) if dims or arr.size == 1 else arr)

    def serialize(self) -> bytes:
        w = Writer()
        a = np.asarray(self.array)
        a = a if a.ndim == 0 else np.ascontiguousarray(a)        # (ascontiguousarray would turn a scalar into [1])
        if a.dtype not in ONNX_TYPES:
            raise ProtoError(f"no ONNX type for {a.dtype}")
        if a.ndim:
            w.packed_varints(1, a.shape)
        w.varint(2, ONNX_TYPES[a.dtype])
        if self.name:
            w.string(8, self.name)
        w.bytes(9, a.astype(a.dtype.newbyteorder("<")).tobytes())
        return w.done()


@dataclass
class Attribute:
    name: str
    value: object = None         # float | int | bytes/str | Tensor | Graph | list of those

    @classmethod
    def parse(cls, buf: bytes) -> "Attribute":
        name, kind = "", 0
        f = i = s = t = g = None
        floats: List[float] = []
        ints: List[int] = []
        strings: List[bytes] = []
        for num, wire, v in fields(buf):
            if num == 1:
                name = v.decode("utf-8")
            elif num == 2:
                f = struct.unpack("<f", v)[0]
            elif num == 3:
                i = _signed(v)
            elif num == 4:
                s = v
            elif num == 5:
                t = Tensor.parse(v)
            elif num == 6:
                g = Graph.parse(v)
            elif num == 7:
                floats += _packed_floats(wire, v)
            elif num == 8:
                ints += _packed_ints(wire, v)
            elif num == 9:
                strings.append(v)
            elif num == 20:
                kind = v
        by_kind = {A_FLOAT: f, A_INT: i, A_STRING: s, A_TENSOR: t, A_GRAPH: g, A_FLOATS: floats, A_INTS: ints, A_STRINGS: strings}
        if kind in by_kind:
            value = by_kind[kind]
        else:                          # writers before the 'type' field: take what is there
            value = next((x for x in (f, i, s, t, g) if x is not None), floats or ints or strings)
        if isinstance(value, bytes):
            value = value.decode("utf-8", errors="replace")
        if value is None:
            value = {A_FLOAT: 0.0, A_INT: 0, A_STRING: ""}.get(kind)
        return cls(name, value)

    def serialize(self) -> bytes:
        w = Writer()
        w.string(1, self.name)
        v = self.value
        if isinstance(v, bool) or isinstance(v, (int, np.integer)):
            w.varint(3, int(v)); w.varint(20, A_INT)
        elif isinstance(v, (float, np.floating)):
            w.float32(2, float(v)); w.varint(20, A_FLOAT)
        elif isinstance(v, (str, bytes)):
            w.bytes(4, v.encode("utf-8") if isinstance(v, str) else v); w.varint(20, A_STRING)
        elif isinstance(v, Tensor):
            w.bytes(5, v.serialize()); w.varint(20, A_TENSOR)
        elif isinstance(v, Graph):
            w.bytes(6, v.serialize()); w.varint(20, A_GRAPH)
        elif isinstance(v, (list, tuple)) and v and isinstance(v[0], (float, np.floating)):
            w.packed_floats(7, [float(x) for x in v]); w.varint(20, A_FLOATS)
        elif isinstance(v, (list, tuple)) and v and isinstance(v[0], (str, bytes)):
            for x in v:
                w.bytes(9, x.encode("utf-8") if isinstance(x, str) else x)
            w.varint(20, A_STRINGS)
        elif isinstance(v, (list, tuple)):
            w.packed_varints(8, v); w.varint(20, A_INTS)
        else:
            raise ProtoError(f"attribute '{self.name}': cannot write a {type(v).__name__}")
        return w.done()


@dataclass
class Node:
    op_type: str
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    attributes: Dict[str, object] = field(default_factory=dict)
    name: str = ""
    domain: str = ""

    @classmethod
    def parse(cls, buf: bytes) -> "Node":
        n = cls("")
        for num, _, v in fields(buf):
            if num == 1:
                n.inputs.append(v.decode("utf-8"))
            elif num == 2:
                n.outputs.append(v.decode("utf-8"))
            elif num == 3:
                n.name = v.decode("utf-8")
            elif num == 4:
                n.op_type = v.decode("utf-8")
            elif num == 5:
                a = Attribute.parse(v)
                n.attributes[a.name] = a.value
            elif num == 7:
                n.domain = v.decode("utf-8")
        return n

    def serialize(self) -> bytes:
        w = Writer()
        for s in self.inputs:
            w.string(1, s)
        for s in self.outputs:
            w.string(2, s)
        if self.name:
            w.string(3, self.name)
        w.string(4, self.op_type)
        for k, v in self.attributes.items():
            w.bytes(5, Attribute(k, v).serialize())
        if self.domain:
            w.string(7, self.domain)
        return w.done()


@dataclass
class ValueInfo:
    name: str
    elem_type: int = FLOAT
    shape: Optional[List[Union[int, str]]] = None

    @classmethod
    def parse(cls, buf: bytes) -> "ValueInfo":
        vi = cls("")
        for num, _, v in fields(buf):
            if num == 1:
                vi.name = v.decode("utf-8")
            elif num == 2:
                for n2, _, t in fields(v):
                    if n2 == 1:                                   # tensor_type
                        for n3, _, x in fields(t):
                            if n3 == 1:
                                vi.elem_type = x
                            elif n3 == 2:
                                vi.shape = []
                                for n4, _, dim in fields(x):
                                    if n4 == 1:
                                        d: Union[int, str] = "?"
                                        for n5, _, dv in fields(dim):
                                            if n5 == 1:
                                                d = _signed(dv)
                                            elif n5 == 2:
                                                d = dv.decode("utf-8")
                                        vi.shape.append(d)
        return vi

    def serialize(self) -> bytes:
        shape = Writer()
        for d in self.shape or []:
            dim = Writer()
            if isinstance(d, str):
                dim.string(2, d)
            else:
                dim.varint(1, d)
            shape.bytes(1, dim.done())
        tensor = Writer()
        tensor.varint(1, self.elem_type)
        if self.shape is not None:
            tensor.bytes(2, shape.done())
        typ = Writer()
        typ.bytes(1, tensor.done())
        w = Writer()
        w.string(1, self.name)
        w.bytes(2, typ.done())
        return w.done()


@dataclass
class Graph:
    name: str = "graph"
    nodes: List[Node] = field(default_factory=list)
    initializers: Dict[str, np.ndarray] = field(default_factory=dict)
    inputs: List[ValueInfo] = field(default_factory=list)
    outputs: List[ValueInfo] = field(default_factory=list)

    @classmethod
    def parse(cls, buf: bytes) -> "Graph":
        g = cls()
        for num, _, v in fields(buf):
            if num == 1:
                g.nodes.append(Node.parse(v))
            elif num == 2:
                g.name = v.decode("utf-8")
            elif num == 5:
                t = Tensor.parse(v)
                g.initializers[t.name] = t.array
            elif num == 11:
                g.inputs.append(ValueInfo.parse(v))
            elif num == 12:
                g.outputs.append(ValueInfo.parse(v))
        return g

    def serialize(self) -> bytes:
        w = Writer()
        for n in self.nodes:
            w.bytes(1, n.serialize())
        w.string(2, self.name)
        for name, arr in self.initializers.items():
            w.bytes(5, Tensor(name, arr).serialize())
        for vi in self.inputs:
            w.bytes(11, vi.serialize())
        for vi in self.outputs:
            w.bytes(12, vi.serialize())
        return w.done()


@dataclass
class Model:
    graph: Graph = field(default_factory=Graph)
    opset: int = 17
    ir_version: int = 8
    producer: str = "idrak_b200"
    opsets: Dict[str, int] = field(default_factory=dict)

    @classmethod
    def parse(cls, buf: bytes) -> "Model":
        m = cls()
        seen_graph = False
        for num, _, v in fields(buf):
            if num == 1:
                m.ir_version = v
            elif num == 2:
                m.producer = v.decode("utf-8")
            elif num == 7:
                m.graph = Graph.parse(v)
                seen_graph = True
            elif num == 8:
                domain, version = "", 0
                for n2, _, x in fields(v):
                    if n2 == 1:
                        domain = x.decode("utf-8")
                    elif n2 == 2:
                        version = x
                m.opsets[domain] = version
        if not seen_graph:
            raise ProtoError("not an ONNX model (no graph)")
        m.opset = m.opsets.get("", m.opset)
        return m

    def serialize(self) -> bytes:
        w = Writer()
        w.varint(1, self.ir_version)
        w.string(2, self.producer)
        w.bytes(7, self.graph.serialize())
        op = Writer()
        op.string(1, "")
        op.varint(2, self.opset)
        w.bytes(8, op.done())
        return w.done()
