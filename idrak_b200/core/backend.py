"""The device contract of the framework and the operation dispatcher over it.

``Backend``           what a device must provide: memory (allocate / upload / download / ranges / copy / copy_to /
                      synchronize / memory report / evict + restore) and the table of operations; two are built in:
                      ``CudaBackend`` (this library's kernels) and ``CpuBackend`` (the PyTorch statements)
``OPERATIONS``        one descriptor per operation: name, the callable of each built-in backend and what happens on a
                      device without a kernel for it - ``host`` (run the CPU statement on downloaded inputs and upload the
                      result), ``composed`` (built from other operations) or ``none`` (refuse by name)
``run(name, ...)``    the dispatcher: a registered plug-in kernel for (operation, device type) wins, else the backend's
                      own kernel, else the descriptor's fallback; every fallback is counted
``capabilities``      optional abilities read once per backend (graph capture, float8 products, segmented attention,
                      fused packed kernels, matrix unit, recurrent kernels, offloading, peer copy, memory report)
``MemoryAccountant``  bytes in use per tag and in total against an optional cap; carved devices
                      (``create_separate_backend``) are a backend with an accountant of their own

Reference: Backend (src/Idrak.Abstraction/Devices/Backend.cs:335, capability interfaces :413-448, MemoryAccountant
:2881, Evict / Restore :948-972, CopyTo :854-871), the generated dispatcher (Devices/Backend.Operations.g.cs), operation
descriptors (Operations/Operation.cs:13-60, KernelSource :77-101), IDeviceKernel plug-ins (src/Idrak.Gpu/Abstractions).
"""
from __future__ import annotations

import dataclasses
import threading
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .registry import SlotTable

HOST, COMPOSED, NONE = "host", "composed", "none"


class DeviceMemoryExceeded(MemoryError):
    def __init__(self, wanted: int, in_use: int, cap: int, tag: str):
        super().__init__(f"allocation of {wanted} bytes ({tag}) exceeds the device cap: {in_use} of {cap} bytes in use")
        self.wanted, self.in_use, self.cap, self.tag = wanted, in_use, cap, tag


class MemoryAccountant:
    """Bytes handed out per tag, the total, the peak, and an optional cap that refuses the allocation that would pass it."""

    def __init__(self, cap_bytes: Optional[int] = None):
        self.cap = cap_bytes
        self.in_use = 0
        self.peak = 0
        self.by_tag: Dict[str, int] = {}
        self._lock = threading.Lock()

    def take(self, nbytes: int, tag: str = "tensor") -> None:
        with self._lock:
            if self.cap is not None and self.in_use + nbytes > self.cap:
                raise DeviceMemoryExceeded(nbytes, self.in_use, self.cap, tag)
            self.in_use += nbytes
            self.peak = max(self.peak, self.in_use)
            self.by_tag[tag] = self.by_tag.get(tag, 0) + nbytes

    def give_back(self, nbytes: int, tag: str = "tensor") -> None:
        with self._lock:
            self.in_use -= nbytes
            self.by_tag[tag] = self.by_tag.get(tag, 0) - nbytes

    def report(self) -> Dict[str, Any]:
        with self._lock:
            return {"in_use": self.in_use, "peak": self.peak, "cap": self.cap,
                    "by_tag": {k: v for k, v in self.by_tag.items() if v}}


@dataclasses.dataclass(frozen=True)
class Operation:
    name: str
    cuda: Optional[Callable] = None        # this library's kernel path (takes CUDA tensors)
    cpu: Optional[Callable] = None         # the PyTorch statement (takes any tensors)
    fallback: str = HOST                   # what a device without a kernel does: host | composed | none
    composed: Optional[Callable] = None    # for fallback == composed: built from other operations via run()
    doc: str = ""


CAPABILITIES = ("graph_capture", "float8_products", "row_attention", "masked_cache_attention", "segmented_attention",
                "fused_packed_kernels", "matrix_unit", "recurrent_kernels", "offloading", "peer_copy", "memory_report",
                "long_lived_allocations")


class Backend:
    """Base device. Subclasses set ``device`` and may override any memory call; operations come from ``OPERATIONS``."""
    kind = "abstract"

    def __init__(self, device: torch.device, accountant: Optional[MemoryAccountant] = None):
        self.device = torch.device(device)
        self.accountant = accountant or MemoryAccountant()
        self._evicted: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._capabilities: Optional[frozenset] = None

    # ------------------------------------------------------------------ memory
    def allocate(self, shape, dtype=torch.float32, tag: str = "tensor") -> torch.Tensor:
        n = 1
        for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)):
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        self.accountant.take(nbytes, tag)
        try:
            t = torch.empty(shape, dtype=dtype, device=self.device)
        except Exception:
            self.accountant.give_back(nbytes, tag)
            raise
        t._idrak_accounted = (nbytes, tag)
        return t

    def give_back(self, t: torch.Tensor) -> None:
        """Return a tensor obtained from ``allocate`` (the storage itself is freed by PyTorch when unreferenced)."""
        rec = getattr(t, "_idrak_accounted", None)
        if rec is not None:
            self.accountant.give_back(*rec)
            t._idrak_accounted = None

    def upload(self, host: torch.Tensor, tag: str = "tensor") -> torch.Tensor:
        out = self.allocate(host.shape, host.dtype, tag)
        out.copy_(host, non_blocking=host.is_pinned())
        return out

    def download(self, t: torch.Tensor) -> torch.Tensor:
        return t.detach().to("cpu")

    def download_range(self, t: torch.Tensor, start: int, count: int) -> torch.Tensor:
        return t.detach().reshape(-1)[start:start + count].to("cpu")

    def upload_range(self, t: torch.Tensor, start: int, host: torch.Tensor) -> None:
        t.reshape(-1)[start:start + host.numel()].copy_(host.reshape(-1))

    def copy(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        dst.copy_(src)

    def copy_2d(self, dst: torch.Tensor, src: torch.Tensor, rows: int, cols: int, dst_ld: int, src_ld: int) -> None:
        d = dst.reshape(-1).as_strided((rows, cols), (dst_ld, 1))
        d.copy_(src.reshape(-1).as_strided((rows, cols), (src_ld, 1)))

    def copy_to(self, t: torch.Tensor, other: "Backend", tag: str = "tensor") -> torch.Tensor:
        """To another backend. Default: through the host; backends that can copy peer to peer override it."""
        return other.upload(self.download(t), tag)

    def create_host_staging(self, nbytes: int) -> torch.Tensor:
        pin = self.device.type == "cuda" and torch.cuda.is_available()
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=pin)

    def synchronize(self) -> None:
        pass

    def memory_usage(self) -> Dict[str, Any]:
        return self.accountant.report()

    # ------------------------------------------------------------------ evict / restore
    def evict(self, t: torch.Tensor) -> None:
        """Move a tensor's contents to the host and free its device storage; ``restore`` brings it back in place, so
        views and autograd references stay valid objects."""
        if id(t) in self._evicted or t.device.type == "cpu":
            return
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
        host.copy_(t)
        if t.is_cuda:
            torch.cuda.current_stream(t.device).synchronize()
        nbytes = t.untyped_storage().nbytes()
        t.untyped_storage().resize_(0)
        self._evicted[id(t)] = (host, torch.tensor(nbytes))

    def restore(self, t: torch.Tensor) -> None:
        rec = self._evicted.pop(id(t), None)
        if rec is None:
            return
        host, nbytes = rec
        t.untyped_storage().resize_(int(nbytes))
        t.copy_(host, non_blocking=True)

    def is_evicted(self, t: torch.Tensor) -> bool:
        return id(t) in self._evicted

    # ------------------------------------------------------------------ capabilities and kernels
    def probe_capabilities(self) -> Iterable[str]:
        return ()

    @property
    def capabilities(self) -> frozenset:
        if self._capabilities is None:          # read once
            self._capabilities = frozenset(c for c in self.probe_capabilities() if c in CAPABILITIES)
        return self._capabilities

    def kernel_for(self, op: Operation) -> Optional[Callable]:
        return None


class CpuBackend(Backend):
    kind = "cpu"

    def __init__(self, accountant: Optional[MemoryAccountant] = None):
        super().__init__(torch.device("cpu"), accountant)

    def probe_capabilities(self):
        return ("memory_report", "offloading", "long_lived_allocations")

    def kernel_for(self, op):
        return op.cpu


class CudaBackend(Backend):
    kind = "cuda"

    def __init__(self, index: int = 0, accountant: Optional[MemoryAccountant] = None):
        super().__init__(torch.device("cuda", index), accountant)

    def probe_capabilities(self):
        from .. import _native
        caps = ["graph_capture", "memory_report", "offloading", "long_lived_allocations", "matrix_unit",
                "row_attention", "masked_cache_attention"]
        if torch.cuda.device_count() > 1:
            caps.append("peer_copy")
        for cap, symbol in (("float8_products", "idrak_gemm_fp8"), ("segmented_attention", "idrak_flash_fwd_ex"),
                            ("fused_packed_kernels", "idrak_skinny_gemm"), ("recurrent_kernels", "idrak_lstm_cell")):
            if _native.has(symbol):
                caps.append(cap)
        return caps

    def kernel_for(self, op):
        return op.cuda

    def synchronize(self):
        torch.cuda.synchronize(self.device)

    def copy_to(self, t, other, tag="tensor"):
        if isinstance(other, CudaBackend) and "peer_copy" in self.capabilities:
            out = other.allocate(t.shape, t.dtype, tag)
            out.copy_(t, non_blocking=True)              # device to device over NVLink, no host hop
            return out
        return super().copy_to(t, other, tag)

    def memory_usage(self):
        rep = super().memory_usage()
        free, total = torch.cuda.mem_get_info(self.device)
        rep.update(device_free=free, device_total=total, torch_allocated=torch.cuda.memory_allocated(self.device),
                   torch_reserved=torch.cuda.memory_reserved(self.device))
        return rep


# --------------------------------------------------------------------------- operations and the dispatcher
def _default_operations(table: SlotTable) -> None:
    from .. import ops
    from ..ops import decode as dops

    def add(name, fn, fallback=HOST, composed=None, doc=""):
        # the public functions of ``ops`` take either device and branch inside; both slots point at them, and a device
        # that is neither gets the fallback
        table.register(name, Operation(name, cuda=fn, cpu=fn, fallback=fallback, composed=composed, doc=doc), "fallback")

    for name in ("gemm", "linear", "mlp_gelu", "mlp_gated", "attention", "qkv_attention", "layer_norm", "rms_norm",
                 "norm_branch", "rope", "gelu", "gated_activation", "embedding", "add", "colsum", "cross_entropy_logits",
                 "token_cross_entropy"):
        add(name, getattr(ops, name))
    for name in ("paged_decode", "kv_write_paged", "argmax_rows", "sample_rows", "norm_rope_kv"):
        if hasattr(dops, name):
            add(name, getattr(dops, name))
    from ..ops import conv as cops, ctc as ctcops, pointwise as pops, recurrent as rops, reduce as redops
    for name in ("unary", "binary", "muladd", "where", "add_rowvec", "dropout"):
        add(name, getattr(pops, name))
    for name in ("softmax", "log_softmax", "scale_mask_softmax", "sum_axis", "broadcast_axis", "permute", "transpose",
                 "gather_rows", "one_hot", "class_match"):
        add(name, getattr(redops, name))
    for name in ("conv2d", "conv1d", "depthwise_conv2d", "max_pool2d", "avg_pool2d"):
        add(name, getattr(cops, name))
    add("ctc_loss", ctcops.ctc_loss)
    for name in ("lstm_cell", "gru_cell", "lstm_layer", "gru_layer"):
        add(name, getattr(rops, name))
    # composed: no kernel of its own anywhere, built from other operations through the dispatcher
    add("silu_mul", None, COMPOSED, composed=lambda backend, gate_up: run("gated_activation", gate_up, "silu", backend=backend),
        doc="SiLU(gate) * up over a packed [.., 2H] tensor")
    add("softmax_cross_entropy", None, COMPOSED,
        composed=lambda backend, logits, targets: run("cross_entropy_logits", logits, targets, backend=backend))
    # none: refused by name on a device without a kernel
    table.register("fp8_product", Operation("fp8_product", cuda=_fp8_product, cpu=None, fallback=NONE,
                                            doc="row-scaled e4m3 product (needs the float8_products capability)"), "fallback")


def _fp8_product(a, b, **kw):
    from ..ops.gemm8 import gemm8
    return gemm8(a, b, **kw)


OPERATIONS: SlotTable = SlotTable("operations", _default_operations)
# plug-in kernels: key (operation name, device type) -> callable; a "shadow" registration wins over the built-in kernel
PLUGIN_KERNELS: SlotTable = SlotTable("plug-in kernels")
FALLBACKS: Dict[str, int] = {}          # operation -> how many calls took the host / composed route
_BACKENDS: Dict[str, Backend] = {}
_LOCK = threading.Lock()


def backend_for(device) -> Backend:
    """The shared backend of a device (``cpu``, ``cuda:0`` ...)."""
    dev = torch.device(device)
    key = f"{dev.type}:{dev.index or 0}" if dev.type == "cuda" else dev.type
    with _LOCK:
        b = _BACKENDS.get(key)
        if b is None:
            b = _BACKENDS[key] = CudaBackend(dev.index or 0) if dev.type == "cuda" else CpuBackend()
        return b


def create_separate_backend(device, cap_bytes: int) -> Backend:
    """A carved device: the same hardware behind an accountant of its own with a memory cap. Allocations through it
    that would pass the cap raise ``DeviceMemoryExceeded`` (how several tenants, or a test, share one GPU)."""
    dev = torch.device(device)
    acc = MemoryAccountant(cap_bytes)
    return CudaBackend(dev.index or 0, acc) if dev.type == "cuda" else CpuBackend(acc)


def register_kernel(operation: str, device_type: str, fn: Callable, policy: str = "shadow"):
    """Plug a kernel in for (operation, device type). Returns the slot; ``slot.remove()`` (or ``with``) takes it out."""
    return PLUGIN_KERNELS.register((operation, device_type), fn, policy)


def _first_tensor_device(args, kwargs) -> torch.device:
    for v in list(args) + list(kwargs.values()):
        if torch.is_tensor(v):
            return v.device
    return torch.device("cpu")


def run(name: str, *args, backend: Optional[Backend] = None, **kwargs):
    """Run an operation by name on the backend of its first tensor argument (or the given one)."""
    op: Optional[Operation] = OPERATIONS.get(name)
    if op is None:
        raise KeyError(f"Operation '{name}' is not registered. Known: {', '.join(sorted(OPERATIONS.keys()))}")
    b = backend or backend_for(_first_tensor_device(args, kwargs))
    plug = PLUGIN_KERNELS.get((name, b.device.type))
    if plug is not None:
        return plug(*args, **kwargs)
    kernel = b.kernel_for(op)
    if kernel is not None:
        return kernel(*args, **kwargs)
    FALLBACKS[name] = FALLBACKS.get(name, 0) + 1
    if op.fallback == COMPOSED and op.composed is not None:
        return op.composed(b, *args, **kwargs)
    if op.fallback == HOST and op.cpu is not None:
        # download, run the host statement, upload the result
        host_args = [b.download(a) if torch.is_tensor(a) else a for a in args]
        host_kw = {k: b.download(v) if torch.is_tensor(v) else v for k, v in kwargs.items()}
        out = op.cpu(*host_args, **host_kw)
        return b.upload(out) if torch.is_tensor(out) and b.device.type != "cpu" else out
    raise NotImplementedError(f"operation '{name}' has no kernel on {b.device} and no fallback")


def operation_report(backend: Optional[Backend] = None) -> List[Dict[str, Any]]:
    """One row per operation: where it would run on this backend."""
    b = backend or backend_for("cuda" if torch.cuda.is_available() else "cpu")
    rows = []
    for name in sorted(OPERATIONS.keys()):
        op = OPERATIONS.get(name)
        source = ("plug-in" if PLUGIN_KERNELS.get((name, b.device.type)) is not None else
                  "device" if b.kernel_for(op) is not None else op.fallback)
        rows.append({"operation": name, "source": source, "fallback": op.fallback, "fallback_calls": FALLBACKS.get(name, 0)})
    return rows
