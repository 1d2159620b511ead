"""Device conformance: does every kernel on this GPU agree with the CPU statement of the same operation?

The scenarios below call the public operations on CPU tensors while a recorder notes each call (operation name,
arguments, result). ``check(device)`` then replays every recorded call on the device - the same argument values,
floating-point tensors cast to the device's compute dtype - and compares the result (and, for differentiable
operations, the gradients of the inputs under a fixed cotangent) with what the CPU gave, inside a tolerance per
operation. An operation the device refuses by ``NotImplementedError`` is reported as skipped, not failed.

Reference: Conformance.Check / CallRecorder / DeviceCases (src/Idrak.Abstraction.Testing/Conformance.cs:33-61,
Devices/CallRecorder.cs, DeviceCases*.cs).
"""
from __future__ import annotations

import dataclasses
import functools
import json
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

# (absolute, relative-to-largest-reference-value) tolerance per operation for a bf16 device against the fp32 host;
# anything not listed takes DEFAULT_TOLERANCE
DEFAULT_TOLERANCE = (2e-2, 2e-2)
TOLERANCES: Dict[str, Tuple[float, float]] = {
    "gemm": (3e-2, 1.5e-2), "linear": (3e-2, 1.5e-2), "mlp_gelu": (4e-2, 2e-2), "mlp_gated": (4e-2, 2e-2),
    "attention": (2e-2, 2e-2), "qkv_attention": (2e-2, 2e-2), "layer_norm": (3e-2, 1e-2), "rms_norm": (3e-2, 1e-2),
    "norm_branch": (3e-2, 1e-2), "rope": (2e-2, 1e-2), "gelu": (1e-2, 1e-2), "gated_activation": (2e-2, 1e-2),
    "embedding": (1e-2, 1e-2), "add": (1e-2, 1e-2), "colsum": (5e-2, 1e-2), "cross_entropy_logits": (2e-2, 1e-2),
    "token_cross_entropy": (3e-2, 1e-2), "argmax_rows": (0.0, 0.0), "paged_decode": (2e-2, 2e-2),
}
# gradients pass through one more rounding than results
GRADIENT_SLACK = 2.5


@dataclasses.dataclass
class RecordedCall:
    """One call of a public operation on the CPU: what went in and what came out."""
    op: str
    args: tuple
    kwargs: dict
    result: Any
    differentiable: bool = False
    scenario: str = ""


@dataclasses.dataclass
class CallOutcome:
    op: str
    scenario: str
    status: str                 # "ok" | "failed" | "skipped" | "error"
    worst: float = 0.0          # largest |device - host| over results and gradients
    allowed: float = 0.0
    detail: str = ""


@dataclasses.dataclass
class ConformanceReport:
    device: str
    outcomes: List[CallOutcome]

    @property
    def ok(self) -> bool:
        return all(o.status in ("ok", "skipped") for o in self.outcomes)

    def counts(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for o in self.outcomes:
            out[o.status] = out.get(o.status, 0) + 1
        return out

    def by_operation(self) -> Dict[str, Dict[str, int]]:
        out: Dict[str, Dict[str, int]] = {}
        for o in self.outcomes:
            out.setdefault(o.op, {}).setdefault(o.status, 0)
            out[o.op][o.status] += 1
        return out

    def to_json(self) -> str:
        return json.dumps({"device": self.device, "ok": self.ok, "counts": self.counts(),
                           "operations": self.by_operation(),
                           "problems": [dataclasses.asdict(o) for o in self.outcomes
                                        if o.status in ("failed", "error")],
                           "skipped": sorted({o.op for o in self.outcomes if o.status == "skipped"})}, indent=1)


def _clone(v):
    if torch.is_tensor(v):
        return v.detach().clone()
    if isinstance(v, (list, tuple)):
        return type(v)(_clone(x) for x in v)
    if isinstance(v, dict):
        return {k: _clone(x) for k, x in v.items()}
    return v


class CallRecorder:
    """Wraps the functions of ``idrak_b200.ops`` for the time of a ``with`` block and keeps every outermost call."""

    def __init__(self, names: Optional[Sequence[str]] = None):
        from .. import ops
        self._ops = ops
        self.names = list(names) if names is not None else [n for n in RECORDED_OPERATIONS if hasattr(ops, n)]
        self.calls: List[RecordedCall] = []
        self._saved: Dict[str, Callable] = {}
        self._depth = 0
        self.scenario = ""

    def _wrap(self, name: str, fn: Callable) -> Callable:
        @functools.wraps(fn)
        def recorded(*args, **kwargs):
            outer = self._depth == 0
            held = (_clone(args), _clone(kwargs)) if outer else None
            self._depth += 1
            try:
                result = fn(*args, **kwargs)
            finally:
                self._depth -= 1
            if outer:
                self.calls.append(RecordedCall(name, held[0], held[1], _clone(result),
                                               name in DIFFERENTIABLE, self.scenario))
            return result
        return recorded

    def __enter__(self):
        for n in self.names:
            self._saved[n] = getattr(self._ops, n)
            setattr(self._ops, n, self._wrap(n, self._saved[n]))
        return self

    def __exit__(self, *exc):
        for n, fn in self._saved.items():
            setattr(self._ops, n, fn)
        self._saved.clear()
        return False


RECORDED_OPERATIONS = ["gemm", "linear", "mlp_gelu", "mlp_gated", "attention", "qkv_attention", "layer_norm", "rms_norm",
                       "norm_branch", "rope", "gelu", "gated_activation", "embedding", "add", "colsum",
                       "cross_entropy_logits", "token_cross_entropy"]
DIFFERENTIABLE = {"linear", "mlp_gelu", "mlp_gated", "attention", "qkv_attention", "layer_norm", "rms_norm",
                  "norm_branch", "rope", "gelu", "gated_activation", "cross_entropy_logits", "token_cross_entropy"}


def _bf16_values(shape, gen, scale=1.0):
    """fp32 tensor holding values that bf16 represents exactly, so host and device start from the same numbers."""
    return (torch.randn(shape, generator=gen) * scale).to(torch.bfloat16).float()


# --------------------------------------------------------------------------- scenarios (run on the CPU, recorded)
def _scenario_products(ops, g):
    for (M, N, K) in ((64, 96, 32), (304, 136, 200), (1024, 768, 256)):      # leading dimensions in whole 16-byte units
        a, b = _bf16_values((M, K), g), _bf16_values((N, K), g, 0.1)
        bias, res = _bf16_values((N,), g, 0.1), _bf16_values((M, N), g)
        ops.gemm(a, b)
        ops.gemm(a, b, bias=bias, residual=res)
        ops.gemm(a, b, bias=bias, act="gelu")
        ops.gemm(a, b, bias=bias, act="gelu_d")
        ops.gemm(a.t().contiguous(), b, a_mn=True)
        ops.gemm(a, b.t().contiguous(), b_mn=True)
        ops.linear(a, b, bias)
        ops.linear(a.reshape(2, M // 2, K), b, None, res.reshape(2, M // 2, N))


def _scenario_feed_forward(ops, g):
    for (T, dim, ff) in ((128, 64, 256), (200, 128, 384)):
        x = _bf16_values((T, dim), g)
        w1, b1 = _bf16_values((ff, dim), g, 0.08), _bf16_values((ff,), g, 0.05)
        w2, b2 = _bf16_values((dim, ff), g, 0.08), _bf16_values((dim,), g, 0.05)
        ops.mlp_gelu(x, w1, b1, w2, b2, x)
        wgu = _bf16_values((2 * ff, dim), g, 0.08)
        for kind in ("silu", "gelu"):
            ops.mlp_gated(x, wgu, None, w2, None, x, kind)
            ops.gated_activation(_bf16_values((T, 2 * ff), g), kind)
        ops.gelu(_bf16_values((T, ff), g))


def _scenario_rows(ops, g):
    for (rows, C) in ((64, 64), (300, 768), (129, 1024), (40, 4096)):
        x = _bf16_values((rows, C), g)
        w, b = _bf16_values((C,), g, 0.2) + 1, _bf16_values((C,), g, 0.2)
        ops.layer_norm(x, w, b, 1e-5)
        ops.rms_norm(x, w, 1e-6)
        ops.norm_branch(x, w, b, 1e-5, False)
        ops.norm_branch(x, w, None, 1e-6, True)
        ops.add(x, _bf16_values((rows, C), g))
        ops.colsum(x)
    ids = torch.randint(0, 500, (3, 70), generator=g)
    ops.embedding(ids, _bf16_values((500, 128), g), _bf16_values((70, 128), g))
    ops.embedding(ids, _bf16_values((500, 128), g))
    for D, rot in ((64, None), (128, 64)):
        x = _bf16_values((90, 4, D), g)
        pos = torch.randint(0, 4000, (90,), generator=g).to(torch.int32)
        ops.rope(x, pos, 10000.0, rot, 1.0)
        ops.rope(x, pos, 500000.0, rot, 0.25)


def _scenario_attention(ops, g):
    for (B, S, H, Hkv, D) in ((1, 128, 2, 2, 64), (2, 200, 4, 2, 64), (1, 384, 4, 1, 128)):
        q, k, v = (_bf16_values((B, S, H, D), g), _bf16_values((B, S, Hkv, D), g), _bf16_values((B, S, Hkv, D), g))
        ops.attention(q, k, v, True)
        ops.attention(q, k, v, False)
        ops.attention(q, k, v, True, None, 96)
        ops.attention(q, k, v, True, None, None, None, 30.0)
        spans = [(0, S // 3), (S // 3, S // 3 + 1), (S // 3 + 1, S)]
        ops.attention(q, k, v, True, None, None, ops.row_starts_from_spans(spans, B, S))
        qkv = _bf16_values((B, S, (H + 2 * Hkv) * D), g)
        ops.qkv_attention(qkv, H, Hkv, D, True, None, 10000.0, None, 1.0, None)
    q, k = _bf16_values((1, 100, 2, 64), g), _bf16_values((1, 333, 2, 64), g)
    ops.attention(q, k, _bf16_values((1, 333, 2, 64), g), False)


def _scenario_losses(ops, g):
    for (rows, V, dim) in ((96, 504, 64), (1000, 4096, 128)):
        logits = _bf16_values((rows, V), g, 2.0)
        tgt = torch.randint(0, V, (rows,), generator=g)
        tgt[::7] = -100
        ops.cross_entropy_logits(logits, tgt)
        h, w = _bf16_values((rows, dim), g), _bf16_values((V + 8, dim), g, 0.1)
        ops.token_cross_entropy(h, w, tgt, V, 256, -100)
        ops.token_cross_entropy(h, w, tgt.clamp(min=0), V, None, None)


SCENARIOS: List[Tuple[str, Callable]] = [
    ("products", _scenario_products), ("feed_forward", _scenario_feed_forward), ("rows", _scenario_rows),
    ("attention", _scenario_attention), ("losses", _scenario_losses),
]


def record_scenarios(names: Optional[Sequence[str]] = None, seed: int = 0) -> List[RecordedCall]:
    """Runs the scenarios on the CPU under the recorder and returns every call they made."""
    from .. import ops
    rec = CallRecorder()
    with rec, torch.no_grad():
        for name, fn in SCENARIOS:
            if names is not None and name not in names:
                continue
            rec.scenario = name
            fn(ops, torch.Generator().manual_seed(seed + len(rec.calls)))
    return rec.calls


# --------------------------------------------------------------------------- replay
def _to_device(v, device, dtype, grads: list):
    if torch.is_tensor(v):
        if v.is_floating_point():
            t = v.to(device=device, dtype=dtype)
            if grads is not None:
                t = t.requires_grad_()
                grads.append(t)
            return t
        return v.to(device)
    if isinstance(v, (list, tuple)):
        return type(v)(_to_device(x, device, dtype, grads) for x in v)
    if isinstance(v, dict):
        return {k: _to_device(x, device, dtype, grads) for k, x in v.items()}
    return v


def _flat(result) -> List[torch.Tensor]:
    if torch.is_tensor(result):
        return [result]
    if isinstance(result, (list, tuple)):
        return [t for r in result for t in _flat(r)]
    return []


def _cotangent(t: torch.Tensor, index: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(1000 + index)
    return torch.randn(t.shape, generator=g).to(torch.bfloat16).float()


def _run(fn: Callable, call: RecordedCall, device, dtype, with_grads: bool):
    leaves: Optional[list] = [] if with_grads else None
    args = _to_device(call.args, device, dtype, leaves)
    kwargs = _to_device(call.kwargs, device, dtype, leaves)
    with torch.enable_grad() if with_grads else torch.no_grad():
        result = fn(*args, **kwargs)
        outs = [t for t in _flat(result) if t.is_floating_point()]
        grads: List[Optional[torch.Tensor]] = []
        if with_grads and outs and any(o.requires_grad for o in outs):
            pairs = [(o, _cotangent(o, i).to(o.device, o.dtype)) for i, o in enumerate(outs) if o.requires_grad]
            got = torch.autograd.grad([p[0] for p in pairs], leaves, [p[1] for p in pairs], allow_unused=True)
            grads = [None if x is None else x.detach().float().cpu() for x in got]
    return [t.detach().float().cpu() if t.is_floating_point() else t.detach().cpu() for t in _flat(result)], grads


def replay(call: RecordedCall, device, dtype: Optional[torch.dtype] = None,
           implementation: Optional[Callable] = None) -> CallOutcome:
    """Runs one recorded call on ``device`` and compares with the host's result (and gradients where the operation is
    differentiable). ``implementation`` replaces the library's function (how a foreign kernel is put to the test)."""
    from .. import ops
    device = torch.device(device)
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    fn = implementation or getattr(ops, call.op)
    abs_tol, rel_tol = TOLERANCES.get(call.op, DEFAULT_TOLERANCE)
    try:
        host_out, host_grads = _run(getattr(ops, call.op), call, "cpu", torch.float32, call.differentiable)
        dev_out, dev_grads = _run(fn, call, device, dtype, call.differentiable)
    except NotImplementedError as e:
        return CallOutcome(call.op, call.scenario, "skipped", detail=str(e)[:200])
    except Exception as e:      # a crash of one call must not end the whole check
        return CallOutcome(call.op, call.scenario, "error", detail=f"{type(e).__name__}: {e}"[:300])
    worst, allowed, detail, bad = 0.0, 0.0, "", False
    pairs = [("result", h, d, 1.0) for h, d in zip(host_out, dev_out)]
    pairs += [("gradient", h, d, GRADIENT_SLACK) for h, d in zip(host_grads, dev_grads) if h is not None and d is not None]
    if len(host_out) != len(dev_out):
        return CallOutcome(call.op, call.scenario, "failed", detail="different number of results")
    for kind, h, d, slack in pairs:
        if h.shape != d.shape:
            return CallOutcome(call.op, call.scenario, "failed", detail=f"{kind} shape {tuple(d.shape)} != {tuple(h.shape)}")
        if not h.is_floating_point():
            if not torch.equal(h, d):
                bad, detail = True, f"{kind}: integer values differ"
            continue
        finite = torch.isfinite(h)
        if not torch.equal(finite, torch.isfinite(d)):
            bad, detail = True, f"{kind}: non-finite values in different places"
            continue
        err = (h[finite] - d[finite]).abs().max().item() if finite.any() else 0.0
        tol = slack * (abs_tol + rel_tol * (h[finite].abs().max().item() if finite.any() else 0.0))
        if err > tol:
            bad, detail = True, f"{kind}: |device - host| = {err:.4g} > {tol:.4g}"
        if err - tol > worst - allowed or allowed == 0.0:
            worst, allowed = err, tol
    return CallOutcome(call.op, call.scenario, "failed" if bad else "ok", worst, allowed, detail)


def check(device="cuda", scenarios: Optional[Sequence[str]] = None, seed: int = 0,
          implementations: Optional[Dict[str, Callable]] = None) -> ConformanceReport:
    """Records the scenarios on the CPU and replays every call on ``device``. ``implementations`` maps operation names
    to functions to test in place of the library's."""
    calls = record_scenarios(scenarios, seed)
    impl = implementations or {}
    outcomes = [replay(c, device, None, impl.get(c.op)) for c in calls]
    dev = torch.device(device)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
        from .. import _native
        try:
            _native.check_status("conformance")
        except Exception as e:
            outcomes.append(CallOutcome("device status", "", "error", detail=str(e)[:300]))
    return ConformanceReport(str(dev), outcomes)
