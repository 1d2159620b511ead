"""ONNX without the onnx package: a hand-written protobuf layer, an exporter for this package's networks and a
runtime that executes imported graphs with tensor ops."""
from . import proto
from .export import GraphWriter, export
from .runtime import OPS, OnnxModule, load
