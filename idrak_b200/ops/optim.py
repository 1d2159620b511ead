"""Fused multi-tensor AdamW / SGD over the native chunk tables, with fp32 master weights.

``FusedAdamW(params)`` keeps for every parameter an fp32 master copy and fp32 moments; the parameter
tensor itself (bf16 on the GPU) is the "shadow" the model computes with and is rewritten by the update
kernel. One step = three launches (sum of squares per chunk, clip factor, update) with no host read;
the gradient norm of the step can be fetched afterwards with :meth:`grad_norm`. Hyper-parameters go to
the device through a pinned block so a recorded CUDA graph keeps following the schedule.

On CPU parameters the same class steps in plain PyTorch fp32 (the formula of ``torch.optim.AdamW``).

State naming for checkpoints follows the reference: ``step``, ``m.{i}``, ``v.{i}`` by parameter index
(src/Idrak.Abstraction/Training/Adam.cs:115-128); the fused path is Adam.ClipAndStep (:80-112).
"""
from __future__ import annotations

import math
from typing import Iterable

import numpy as np
import torch

from .. import _native
from ._util import scratch, stream_ptr

H_LR, H_B1, H_B2, H_EPS, H_BC1, H_BC2, H_CLIP, H_NORM, H_MAXNORM, H_GSCALE, H_COUNT = range(11)

_TENSOR_DT = np.dtype([("master", "<u8"), ("shadow", "<u8"), ("grad", "<u8"), ("m", "<u8"), ("v", "<u8"),
                       ("n", "<i8"), ("wd", "<f4"), ("grad_fp32", "<i4")])
_CHUNK_DT = np.dtype([("tensor", "<i4"), ("pad", "<i4"), ("first", "<i8")])


class FusedOptimizerBase:
    """Parameter groups, master weights and the device tables shared by AdamW and SGD."""

    def __init__(self, params: Iterable, lr: float, weight_decay: float, max_grad_norm: float = 0.0):
        groups = list(params)
        if groups and not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        self.param_groups = []
        for g in groups:
            g = dict(g)
            g["params"] = [p for p in g["params"]]
            g.setdefault("lr", lr)
            g.setdefault("weight_decay", weight_decay)
            self.param_groups.append(g)
        self.params = [p for g in self.param_groups for p in g["params"]]
        self._wd = [g["weight_decay"] for g in self.param_groups for _ in g["params"]]
        self.lr = lr
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.grad_scale = 1.0
        self.master: list[torch.Tensor] = []
        self._tables = None
        self._table_key = None
        self._hyper_host = None
        self._hyper_dev = None
        self.cuda = bool(self.params) and self.params[0].is_cuda
        for p in self.params:
            self.master.append(p.detach().float().clone() if p.dtype != torch.float32 else p.detach())

    # ------------------------------------------------------------------ torch.optim-like surface
    def zero_grad(self, set_to_none: bool = False):
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    def set_lr(self, lr: float):
        self.lr = lr
        for g in self.param_groups:
            g["lr"] = lr

    def grad_norm(self) -> float:
        """Gradient norm seen by the last step (reads one float from the device)."""
        if self._hyper_dev is None:
            return 0.0
        return float(self._hyper_dev[H_NORM].item())

    # ------------------------------------------------------------------ device tables
    def _state_tensors(self, i):  # -> (m, v)
        raise NotImplementedError

    def _ensure_grads(self):
        for p in self.params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)

    def _build_tables(self):
        self._ensure_grads()
        key = tuple((p.data_ptr(), p.grad.data_ptr()) for p in self.params)
        if self._tables is not None and key == self._table_key:
            return self._tables
        lib = _native.lib()
        assert lib.idrak_opt_tensor_bytes() == _TENSOR_DT.itemsize
        assert lib.idrak_opt_chunk_bytes() == _CHUNK_DT.itemsize
        chunk = lib.idrak_opt_chunk_elems()
        tens = np.zeros(len(self.params), dtype=_TENSOR_DT)
        chunks = []
        for i, p in enumerate(self.params):
            m, v = self._state_tensors(i)
            g = p.grad
            assert p.is_contiguous() and g.is_contiguous()
            tens[i] = (self.master[i].data_ptr(), 0 if p.dtype == torch.float32 else p.data_ptr(), g.data_ptr(),
                       m.data_ptr(), v.data_ptr() if v is not None else 0, p.numel(), self._wd[i],
                       1 if g.dtype == torch.float32 else 0)
            for first in range(0, p.numel(), chunk):
                chunks.append((i, 0, first))
        ch = np.array(chunks, dtype=_CHUNK_DT)
        dev = self.params[0].device
        t_dev = torch.from_numpy(tens.view(np.uint8).copy()).to(dev)
        c_dev = torch.from_numpy(ch.view(np.uint8).copy()).to(dev)
        partial = torch.empty(max(1, len(chunks)), dtype=torch.float32, device=dev)
        self._tables = (t_dev, c_dev, len(chunks), partial)
        self._table_key = key
        if self._hyper_dev is None:
            # a ring of pinned blocks: the copy of step t may still be pending when the host prepares t+1
            self._hyper_host = torch.zeros(16, H_COUNT, dtype=torch.float32).pin_memory()
            self._hyper_dev = torch.zeros(H_COUNT, dtype=torch.float32, device=dev)
        return self._tables

    def _hyper_values(self) -> dict:
        raise NotImplementedError

    def advance_for_replay(self):
        """A recorded CUDA graph replays the launches of ``step``; the host side of a step (count the step,
        refresh the pinned hyper-parameter block the graph copies from) is this call."""
        self.step_count += 1
        h = self._hyper_host[0]
        for k, v in self._hyper_values().items():
            h[k] = v

    def _upload_hyper(self, values: dict):
        # under graph capture the copy node must always read the same pinned block
        slot = 0 if torch.cuda.is_current_stream_capturing() else 1 + self.step_count % 15
        h = self._hyper_host[slot]
        for k, v in values.items():
            h[k] = v
        # clip scale / norm slots are written by the device; do not overwrite them mid-step
        self._hyper_dev[:H_CLIP].copy_(h[:H_CLIP], non_blocking=True)
        self._hyper_dev[H_MAXNORM:].copy_(h[H_MAXNORM:], non_blocking=True)


class FusedAdamW(FusedOptimizerBase):
    def __init__(self, params, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                 max_grad_norm: float = 0.0, zero_grad_in_step: bool = False):
        super().__init__(params, lr, weight_decay, max_grad_norm)
        self.betas, self.eps = betas, eps
        self.zero_grad_in_step = zero_grad_in_step
        self.m = [torch.zeros_like(w, dtype=torch.float32) for w in self.master]
        self.v = [torch.zeros_like(w, dtype=torch.float32) for w in self.master]

    def _state_tensors(self, i):
        return self.m[i], self.v[i]

    @torch.no_grad()
    def step(self, extra_sumsq: torch.Tensor | None = None):
        self.step_count += 1
        b1, b2 = self.betas
        bc1 = 1.0 - b1 ** self.step_count
        bc2 = 1.0 - b2 ** self.step_count
        if not self.cuda:
            return self._step_cpu(bc1, bc2, extra_sumsq)
        lib = _native.lib()
        t_dev, c_dev, n_chunks, partial = self._build_tables()
        self._upload_hyper(self._hyper_values())
        s = stream_ptr()
        rc = lib.idrak_opt_grad_norm(t_dev.data_ptr(), c_dev.data_ptr(), n_chunks, partial.data_ptr(),
                                     extra_sumsq.data_ptr() if extra_sumsq is not None else None,
                                     self._hyper_dev.data_ptr(), s)
        _native.check(rc, "idrak_opt_grad_norm")
        rc = lib.idrak_opt_adamw(t_dev.data_ptr(), c_dev.data_ptr(), n_chunks, self._hyper_dev.data_ptr(),
                                 int(self.zero_grad_in_step), s)
        _native.check(rc, "idrak_opt_adamw")

    def _hyper_values(self) -> dict:
        b1, b2 = self.betas
        return {H_LR: self.lr, H_B1: b1, H_B2: b2, H_EPS: self.eps, H_BC1: 1.0 - b1 ** self.step_count,
                H_BC2: 1.0 - b2 ** self.step_count, H_MAXNORM: self.max_grad_norm, H_GSCALE: self.grad_scale}

    def _step_cpu(self, bc1, bc2, extra_sumsq=None):
        b1, b2 = self.betas
        live = [i for i, p in enumerate(self.params) if p.grad is not None]
        grads = [self.params[i].grad.float() for i in live]
        if self.grad_scale != 1.0:
            grads = [g * self.grad_scale for g in grads]
        sq = float(torch.stack(torch._foreach_norm(grads)).pow(2).sum()) if grads else 0.0
        if extra_sumsq is not None:
            sq += float(extra_sumsq.sum())
        norm = math.sqrt(sq)
        self._last_norm = norm
        if self.max_grad_norm > 0 and norm > self.max_grad_norm:
            grads = torch._foreach_mul(grads, self.max_grad_norm / (norm + 1e-6))
        ms, vs, ws = [self.m[i] for i in live], [self.v[i] for i in live], [self.master[i] for i in live]
        torch._foreach_mul_(ms, b1)
        torch._foreach_add_(ms, grads, alpha=1 - b1)
        torch._foreach_mul_(vs, b2)
        torch._foreach_addcmul_(vs, grads, grads, value=1 - b2)
        torch._foreach_mul_(ws, [1 - self.lr * self._wd[i] for i in live])
        denom = torch._foreach_sqrt(vs)
        torch._foreach_div_(denom, math.sqrt(bc2))
        torch._foreach_add_(denom, self.eps)
        torch._foreach_addcdiv_(ws, ms, denom, value=-self.lr / bc1)
        for i in live:
            p, w = self.params[i], self.master[i]
            if w.data_ptr() != p.data_ptr():
                p.copy_(w.to(p.dtype))
            if self.zero_grad_in_step:
                p.grad.zero_()

    def grad_norm(self) -> float:
        if not self.cuda:
            return getattr(self, "_last_norm", 0.0)
        return super().grad_norm()

    # ------------------------------------------------------------------ checkpoint state (reference naming)
    def state_dict(self) -> dict:
        out = {"step": torch.tensor(float(self.step_count))}
        for i in range(len(self.params)):
            out[f"m.{i}"] = self.m[i].detach().cpu()
            out[f"v.{i}"] = self.v[i].detach().cpu()
        return out

    def load_state_dict(self, state: dict):
        self.step_count = int(float(state["step"]))
        for i in range(len(self.params)):
            self.m[i].copy_(state[f"m.{i}"].reshape(self.m[i].shape))
            self.v[i].copy_(state[f"v.{i}"].reshape(self.v[i].shape))
        for i, p in enumerate(self.params):
            if self.master[i].data_ptr() != p.data_ptr():
                pass  # masters are restored by the caller from fp32 weights when present

    def sync_master_from_params(self):
        for i, p in enumerate(self.params):
            if self.master[i].data_ptr() != p.data_ptr():
                self.master[i].copy_(p.detach().float())


class FusedSGD(FusedOptimizerBase):
    def __init__(self, params, lr: float = 1e-2, momentum: float = 0.0, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.0, zero_grad_in_step: bool = False):
        super().__init__(params, lr, weight_decay, max_grad_norm)
        self.momentum = momentum
        self.zero_grad_in_step = zero_grad_in_step
        self.m = [torch.zeros_like(w, dtype=torch.float32) for w in self.master]

    def _state_tensors(self, i):
        return self.m[i], None

    @torch.no_grad()
    def step(self, extra_sumsq=None):
        self.step_count += 1
        if not self.cuda:
            for i, p in enumerate(self.params):
                if p.grad is None:
                    continue
                w = self.master[i]
                g = p.grad.float() * self.grad_scale + self._wd[i] * w
                if self.momentum:
                    self.m[i].mul_(self.momentum).add_(g)
                    g = self.m[i]
                w.add_(g, alpha=-self.lr)
                if w.data_ptr() != p.data_ptr():
                    p.copy_(w.to(p.dtype))
            return
        lib = _native.lib()
        t_dev, c_dev, n_chunks, partial = self._build_tables()
        self._upload_hyper(self._hyper_values())
        s = stream_ptr()
        _native.check(lib.idrak_opt_grad_norm(t_dev.data_ptr(), c_dev.data_ptr(), n_chunks, partial.data_ptr(),
                                              extra_sumsq.data_ptr() if extra_sumsq is not None else None,
                                              self._hyper_dev.data_ptr(), s), "idrak_opt_grad_norm")
        _native.check(lib.idrak_opt_sgd(t_dev.data_ptr(), c_dev.data_ptr(), n_chunks, self._hyper_dev.data_ptr(),
                                        float(self.momentum), int(self.zero_grad_in_step), s), "idrak_opt_sgd")

    def _hyper_values(self) -> dict:
        return {H_LR: self.lr, H_MAXNORM: self.max_grad_norm, H_GSCALE: self.grad_scale}

    def state_dict(self):
        out = {"step": torch.tensor(float(self.step_count))}
        for i in range(len(self.params)):
            out[f"m.{i}"] = self.m[i].detach().cpu()
        return out

    def load_state_dict(self, state):
        self.step_count = int(float(state["step"]))
        for i in range(len(self.params)):
            self.m[i].copy_(state[f"m.{i}"].reshape(self.m[i].shape))
