"""Scopes that change how work inside them runs: product precision, activation memory policy, tensor lifetime, and a
captured compute graph.

* ``mixed_precision("bfloat16")`` - products inside run with operands rounded to that type (autocast for library
  modules; this package's own layers follow their parameters' dtype). ``IDRAK_MATMUL`` sets the process default.
* ``activation_memory(model, "checkpoint_blocks" | "held")`` - switches a decoder between keeping block activations
  and recomputing them in backward.
* ``TensorScope`` - frees what was allocated inside on exit (the caching allocator makes this a no-op except for an
  optional cache trim).
* ``ComputeGraph`` - capture a function over static inputs as a CUDA graph, replay it with new input values.

Reference: MixedPrecision.Use (src/Idrak.Abstraction/Tensors/MixedPrecision.cs:54), ActivationMemory.CheckpointBlocks /
Recompute / CompressToBFloat16 (ActivationMemory.cs), TensorScope.cs, ComputeGraph.Capture / Replay (ComputeGraph.cs).
"""
from __future__ import annotations

import contextlib
import os
from typing import Callable, Optional, Sequence

import torch

_KINDS = {"float32": None, "f32": None, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
          "f16": torch.float16}
# Products in 8-bit floats need the fp8 GEMM (ops/gemm8.py); a scope asking for them says so by name instead of
# running bf16 under another label, and the request is counted like the reference counts reduced-precision fallbacks
# (src/Idrak.Gpu/ReducedPrecision.cs, CudaBackend.cs:1385-1388).
_FLOAT8 = ("float8", "f8")
fallbacks = {"float8_to_bfloat16": 0}
_current = [os.environ.get("IDRAK_MATMUL", "float32").lower()]


def product_precision() -> str:
    """The precision products run at in the current scope."""
    return _current[-1]


@contextlib.contextmanager
def mixed_precision(kind: str):
    k = kind.lower()
    if k in _FLOAT8:
        import warnings
        fallbacks["float8_to_bfloat16"] += 1
        warnings.warn("mixed_precision('float8'): layers built from idrak_b200 modules have no 8-bit product path inside "
                      "autocast; products in this scope run in bfloat16 (use ops.gemm8 for an explicit fp8 product)",
                      RuntimeWarning, stacklevel=3)
        k = "bfloat16"
    if k not in _KINDS:
        raise ValueError(f"unknown precision '{kind}'; known: {', '.join(sorted(set(_KINDS)))}")
    _current.append(k)
    dtype = _KINDS[k]
    try:
        if dtype is None:
            with torch.autocast("cuda", enabled=False), torch.autocast("cpu", enabled=False):
                yield
        else:
            with torch.autocast("cuda", dtype=dtype), torch.autocast("cpu", dtype=torch.bfloat16):
                yield
    finally:
        _current.pop()


@contextlib.contextmanager
def activation_memory(model: torch.nn.Module, policy: str):
    """``held`` keeps every block's activations; ``checkpoint_blocks`` keeps block inputs only and re-runs each block
    in backward. Applies to modules that expose ``checkpoint_blocks`` (the decoder and its parallel variants)."""
    if policy not in ("held", "checkpoint_blocks"):
        raise ValueError("policy must be 'held' or 'checkpoint_blocks'")
    touched = [(m, m.checkpoint_blocks) for m in model.modules() if hasattr(m, "checkpoint_blocks")]
    for m, _ in touched:
        m.checkpoint_blocks = policy == "checkpoint_blocks"
    try:
        yield
    finally:
        for m, old in touched:
            m.checkpoint_blocks = old


class compress_saved_to_bfloat16:
    """Scope: float32 tensors that autograd saves for the backward pass are kept as bfloat16 and widened again when the
    backward pass asks for them - half the activation memory of an fp32 model for one rounding of what backward reads.
    Tensors below ``min_elements``, non-float32 tensors and parameters (saved by reference, not copied) pass through.
    ``stats`` counts what was compressed.

    Reference: ActivationMemory.CompressToBFloat16 (src/Idrak.Abstraction/Tensors/ActivationMemory.cs:23)."""

    def __init__(self, min_elements: int = 1024):
        self.min_elements = min_elements
        self.stats = {"tensors": 0, "bytes_saved": 0}
        self._hooks = None

    def _pack(self, t: torch.Tensor):
        if (t.dtype != torch.float32 or t.numel() < self.min_elements or isinstance(t, torch.nn.Parameter)
                or not t.is_floating_point()):
            return t
        self.stats["tensors"] += 1
        self.stats["bytes_saved"] += t.numel() * 2
        return ("bf16", t.to(torch.bfloat16))

    @staticmethod
    def _unpack(packed):
        if isinstance(packed, tuple) and len(packed) == 2 and packed[0] == "bf16":
            return packed[1].float()
        return packed

    def __enter__(self):
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        return self._hooks.__exit__(*exc)


@contextlib.contextmanager
def recompute(model: torch.nn.Module, what: str = "feed_forward"):
    """Scope: the named part of every block is re-run in the backward pass instead of keeping its inner activations
    (``feed_forward``: the [tokens, ff] intermediates, the largest activations of a block; ``attention``; ``blocks``:
    whole blocks, the same as ``activation_memory(model, "checkpoint_blocks")``).

    Reference: ActivationMemory.Recompute (src/Idrak.Abstraction/Tensors/ActivationMemory.cs:23)."""
    from .checkpointing import checkpoint
    if what == "blocks":
        with activation_memory(model, "checkpoint_blocks"):
            yield
        return
    attr = {"feed_forward": "mlp", "attention": "attn"}.get(what)
    if attr is None:
        raise ValueError("what must be 'feed_forward', 'attention' or 'blocks'")
    wrapped = []
    for blk in getattr(model, "blocks", []):
        part = getattr(blk, attr, None)
        if part is None:
            continue
        original = part.forward

        def recomputed(*args, _f=original, **kwargs):
            if not torch.is_grad_enabled() or not any(torch.is_tensor(a) and a.requires_grad for a in args):
                return _f(*args, **kwargs)
            return checkpoint(_f, *args, **kwargs)
        part.forward = recomputed
        wrapped.append((part, original))
    try:
        yield
    finally:
        for part, original in wrapped:
            part.forward = original


class TensorScope:
    """``with TensorScope() as scope: ...`` - arena-style disposal. Tensors handed to ``scope.own(t)`` lose their storage
    when the scope ends even if references to them remain (the reference's scope frees everything allocated inside
    it); ``scope.keep(t)`` takes one out again so it survives. ``trim=True`` also returns cached blocks to the
    driver on exit.

    Reference: TensorScope (src/Idrak.Abstraction/Tensors/TensorScope.cs:23)."""

    def __init__(self, trim: bool = False):
        self.trim = trim
        self._owned = {}

    def own(self, t: torch.Tensor) -> torch.Tensor:
        self._owned[id(t)] = t
        return t

    def keep(self, t: torch.Tensor) -> torch.Tensor:
        self._owned.pop(id(t), None)
        return t

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for t in self._owned.values():
            try:
                t.untyped_storage().resize_(0)          # the memory goes now, whoever still holds the object
            except RuntimeError:
                pass                                     # storage shared with something not resizable: left to refcounts
        self._owned.clear()
        if self.trim and torch.cuda.is_available():
            torch.cuda.empty_cache()
        return False


class ComputeGraph:
    """A function over fixed-shape device inputs, recorded once and replayed.

        g = ComputeGraph.capture(fn, example_a, example_b)
        out = g.replay(new_a, new_b)          # copies the new values into the recorded inputs, launches the graph
    """

    def __init__(self, graph, inputs: Sequence[torch.Tensor], outputs):
        self.graph, self.inputs, self.outputs = graph, list(inputs), outputs
        self.replays = 0

    @classmethod
    def capture(cls, fn: Callable, *inputs: torch.Tensor, warmup: int = 2) -> "ComputeGraph":
        if not inputs or not all(t.is_cuda for t in inputs):
            raise ValueError("capture takes CUDA tensors")
        static = [t.clone() for t in inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):          # lazy initialisation (kernel attributes, workspaces) happens here
                fn(*static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outputs = fn(*static)
        return cls(graph, static, outputs)

    def replay(self, *inputs: torch.Tensor):
        if len(inputs) != len(self.inputs):
            raise ValueError(f"the graph was recorded with {len(self.inputs)} inputs")
        for dst, src in zip(self.inputs, inputs):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError("replay inputs must match the recorded shapes and types")
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.outputs
