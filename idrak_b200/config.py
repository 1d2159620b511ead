"""Process-wide settings: one table of environment variables with types, defaults and meaning.

``settings.get("IDRAK_TP_MULTIMEM")`` reads and validates a variable; ``describe()`` renders the table (the
``idrak config`` command prints it). A value that does not parse is an error that names the variable, never a
silent default.

Reference: the environment table of the reference (src/Idrak.Abstraction/Configuration/EnvironmentSettings.cs) and
``idrak config`` (src/Idrak.Cli.Commands/Commands/ConfigCommands.cs).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional


def _bool(text: str) -> bool:
    t = text.strip().lower()
    if t in ("1", "true", "yes", "on"):
        return True
    if t in ("0", "false", "no", "off", ""):
        return False
    raise ValueError("expected 0/1, true/false, yes/no or on/off")


def _size(text: str) -> int:
    """Bytes with a power-of-1,024 unit: 512M, 2G, 64K, or a plain integer."""
    t = text.strip().upper().rstrip("B")
    units = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40}
    if t and t[-1] in units:
        return int(float(t[:-1]) * units[t[-1]])
    return int(t)


@dataclass(frozen=True)
class Setting:
    name: str
    kind: str                    # bool | int | float | size | text | choice
    default: Any
    help: str
    choices: tuple = ()

    def parse(self, text: str) -> Any:
        try:
            if self.kind == "bool":
                return _bool(text)
            if self.kind == "int":
                return int(text)
            if self.kind == "float":
                return float(text)
            if self.kind == "size":
                return _size(text)
            if self.kind == "choice":
                if text not in self.choices:
                    raise ValueError(f"expected one of {', '.join(self.choices)}")
                return text
            return text
        except ValueError as e:
            raise ValueError(f"{self.name}={text!r}: {e}") from None


TABLE: List[Setting] = [
    Setting("IDRAK_BENCH_GRAPH", "bool", True, "bench.py: replay the training step as a CUDA graph"),
    Setting("IDRAK_BENCH_DP", "choice", "fused", "bench.py: data-parallel path", ("fused", "nccl")),
    Setting("IDRAK_TP_MULTIMEM", "bool", True, "tensor parallel: use NVSwitch multicast stores / reducing loads when "
                                               "the machine offers them"),
    Setting("IDRAK_TP_PUSH_CTAS", "int", 16, "tensor parallel: CTAs of the all-gather->GEMM kernel that move rows"),
    Setting("IDRAK_PREFILL_CHUNK", "int", 8192, "serving: most prompt tokens computed in one prefill step"),
    Setting("IDRAK_KV_FRACTION", "float", 0.8, "serving: share of the free device memory given to the KV cache"),
    Setting("IDRAK_MAX_BATCH", "int", 64, "serving: most sequences decoded together"),
    Setting("IDRAK_QUEUE_LIMIT", "int", 0, "serving: most requests waiting per model (0 = unbounded)"),
    Setting("IDRAK_REQUEST_TIMEOUT", "float", 0.0, "serving: seconds a request may wait in the queue (0 = forever)"),
    Setting("IDRAK_KEEP_ALIVE", "float", 300.0, "serving: seconds an idle model stays loaded (0 = forever)"),
    Setting("IDRAK_WORKSPACE", "size", 256 << 20, "largest scratch buffer an op may keep between calls"),
    Setting("IDRAK_TELEMETRY", "text", "", "telemetry levels to record, comma separated (step, kernel, comm, memory)"),
    Setting("IDRAK_TELEMETRY_FILE", "text", "", "write telemetry events to this JSON-lines file"),
    Setting("IDRAK_HOME", "text", os.path.join(os.path.expanduser("~"), ".idrak"), "models, runs and aliases live here"),
    Setting("IDRAK_STOP_FILE", "text", "", "training stops cleanly at the next step when this file appears"),
    Setting("IDRAK_CUDA_DEBUG", "bool", False, "synchronise after every native launch and name the call that failed"),
    Setting("IDRAK_GEMM_PAIR", "choice", "1", "large one-pass GEMMs on CTA pairs (256 x 256 tiles, cta_group::2): 0 never, "
            "1 where it measured faster, 2 wherever it can run", ("0", "1", "2")),
    Setting("IDRAK_DP_DEBUG", "bool", False, "data parallel: record where a duplicate gradient-ready signal came from"),
    Setting("IDRAK_AUTOTUNE", "bool", False, "time the candidates the first time a shape class needs a choice and keep the winner"),
    Setting("IDRAK_TUNING_CACHE", "text", "", "file of measured decisions (default: tuning.json under IDRAK_HOME)"),
    Setting("IDRAK_MATMUL", "choice", "float32", "precision of products in library modules outside a mixed_precision scope",
            ("float32", "bfloat16", "float16", "float8")),
    Setting("IDRAK_TOKENIZER", "choice", "library", "runtime for tokenizer.json files: the tokenizers library, or this package's "
            "own BPE / WordPiece / Unigram runtime (native merge engine)", ("library", "own")),
    Setting("IDRAK_DEVICE", "text", "", "default device of Device.default() and the command line (cpu, cuda, cuda:N, gpu:N)"),
    Setting("IDRAK_PLUGINS", "text", "", "comma-separated plug-in modules imported by load_plugins()"),
    Setting("IDRAK_NORM_BULK", "bool", True, "norm backward: the pipelined kernel (rows staged through shared memory by bulk copies)"),
    Setting("IDRAK_XENT_BULK", "bool", True, "cross-entropy: the pipelined one-pass kernel when a row fits shared memory"),
    Setting("IDRAK_FEW_ROW_DECODE", "bool", True, "serving: decode steps of up to 64 sequences on the few-row projection kernels"),
    Setting("IDRAK_TP_AR", "choice", "auto", "tensor-parallel serving: all-reduce of the partial rows (auto picks one-shot "
            "up to 256 rows)", ("auto", "oneshot", "twoshot", "nccl")),
    Setting("IDRAK_WAIT_BUDGET_NS", "int", 2_000_000_000, "how long a device-side wait (barrier, flag) may spin before it "
            "records where it gave up and returns"),
    Setting("IDRAK_NVCC", "text", "", "compiler used by python -m idrak_b200.build (default: nvcc on PATH or /usr/local/cuda)"),
    Setting("IDRAK_B200_LIB", "text", "", "load this native library instead of lib/libidrak_b200.so"),
    Setting("IDRAK_TP_FEW_ROW_DECODE", "bool", True, "tensor-parallel serving: decode steps of up to 64 sequences on the few-row kernels"),
    Setting("IDRAK_PDL", "bool", True, "few-row decode products are launched programmatically dependent on the kernel "
                                       "before them (their set-up overlaps its tail); 0 launches them the ordinary way"),
    Setting("IDRAK_SKINNY_SPLITS", "choice", "", "few-row products: force the number of CTAs that share K (for measurements)",
            ("", "1", "2", "4", "8")),
    Setting("IDRAK_B200_AUTOBUILD", "bool", False, "build the native library on first use when it is missing"),
    Setting("IDRAK_REFERENCE_DATA", "text", "", "tests: folder with the reference project's test fixtures"),
    Setting("IDRAK_COMM_CANARIES", "bool", True, "communicator: check the guard bands of symmetric buffers at close"),
]
_BY_NAME: Dict[str, Setting] = {s.name: s for s in TABLE}


class Settings:
    def __init__(self, environ: Optional[Dict[str, str]] = None):
        self.environ = environ if environ is not None else os.environ
        self._overrides: Dict[str, Any] = {}

    def get(self, name: str) -> Any:
        if name not in _BY_NAME:
            raise KeyError(f"unknown setting {name}; known: {', '.join(sorted(_BY_NAME))}")
        if name in self._overrides:
            return self._overrides[name]
        s = _BY_NAME[name]
        raw = self.environ.get(name)
        return s.default if raw is None else s.parse(raw)

    def set(self, name: str, value: Any) -> None:
        s = _BY_NAME[name] if name in _BY_NAME else None
        if s is None:
            raise KeyError(f"unknown setting {name}")
        self._overrides[name] = s.parse(value) if isinstance(value, str) else value

    def validate(self) -> List[str]:
        """Problems with the current environment: unparsable values and unknown IDRAK_* names."""
        problems = []
        for key, raw in self.environ.items():
            if not key.startswith("IDRAK_"):
                continue
            if key not in _BY_NAME:
                problems.append(f"{key}: not a setting of this package")
                continue
            try:
                _BY_NAME[key].parse(raw)
            except ValueError as e:
                problems.append(str(e))
        return problems


settings = Settings()


def get(name: str) -> Any:
    """The current value of a setting (environment, or an override made with ``settings.set``)."""
    return settings.get(name)


def describe(current: Optional[Settings] = None) -> str:
    cur = current or settings
    rows = [("name", "type", "default", "now", "meaning")]
    for s in TABLE:
        try:
            now = cur.get(s.name)
        except ValueError as e:
            now = f"invalid ({e})"
        rows.append((s.name, s.kind if not s.choices else "|".join(s.choices), str(s.default), str(now), s.help))
    widths = [max(len(r[i]) for r in rows) for i in range(4)]
    return "\n".join("  ".join(r[i].ljust(widths[i]) for i in range(4)) + "  " + r[4] for r in rows)
