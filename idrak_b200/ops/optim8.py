"""AdamW with 8-bit moments (2 bytes of optimizer state per parameter instead of 8).

Both moments are stored as one byte per value, scaled per block of 256 values by the block's largest magnitude;
a byte indexes a fixed non-linear map that is denser near zero. The update de-quantises, steps in fp32 and
re-quantises inside one kernel (``csrc/adam8.cu``); on CPU tensors the same arithmetic runs in PyTorch.

Reference: EightBitMoments and the adam8_f32 kernel (src/Idrak.Abstraction/Devices/Backend.cs:2099,
src/Idrak.Gpu/Cuda/PtxKernels.Rows.cs:258).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Iterable, List

import torch

from .. import _native
from ._util import stream_ptr

BLOCK = 256
_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    _native.bind("idrak_adam8_step", i, [vp, vp, vp, i, vp, vp, vp, vp, ll, f, f, f, f, f, f, f, f, vp, vp])
    _BOUND = True


# ---- the maps, as PyTorch (CPU path and test oracle)
def signed_value(codes: torch.Tensor) -> torch.Tensor:
    x = (codes.float() - 127.5) / 127.5
    return x * x.abs()


def signed_code(y: torch.Tensor) -> torch.Tensor:
    x = torch.sign(y) * torch.sqrt(y.abs())
    return torch.clamp(torch.round(x * 127.5 + 127.5), 0, 255).to(torch.uint8)


def unsigned_value(codes: torch.Tensor) -> torch.Tensor:
    x = codes.float() / 255.0
    return x * x


def unsigned_code(y: torch.Tensor) -> torch.Tensor:
    x = torch.sqrt(y.clamp_min(0)) * 255.0
    c = torch.ceil(x - 1e-4)
    c = torch.where(y > 0, c.clamp_min(1), torch.zeros_like(c))
    return c.clamp(0, 255).to(torch.uint8)


class Adam8bit:
    def __init__(self, params: Iterable, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 0.0):
        groups = list(params)
        if groups and not isinstance(groups[0], dict):
            groups = [{"params": groups, "weight_decay": weight_decay}]
        self.params: List[torch.Tensor] = []
        self._wd: List[float] = []
        for g in groups:
            for p in g["params"]:
                if p.requires_grad:
                    self.params.append(p)
                    self._wd.append(float(g.get("weight_decay", weight_decay)))
        self.lr, self.betas, self.eps, self.max_grad_norm = lr, betas, eps, max_grad_norm
        self.step_count = 0
        self.master, self.m8, self.v8, self.m_absmax, self.v_absmax = [], [], [], [], []
        for p in self.params:
            n = p.numel()
            blocks = (n + BLOCK - 1) // BLOCK
            self.master.append(p.detach().float().clone() if p.dtype != torch.float32 else p.detach())
            self.m8.append(torch.full((n,), 128, dtype=torch.uint8, device=p.device))
            self.v8.append(torch.zeros(n, dtype=torch.uint8, device=p.device))
            self.m_absmax.append(torch.zeros(blocks, dtype=torch.float32, device=p.device))
            self.v_absmax.append(torch.zeros(blocks, dtype=torch.float32, device=p.device))

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for ts in (self.m8, self.v8, self.m_absmax, self.v_absmax) for t in ts)

    def zero_grad(self, set_to_none: bool = False):
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        clip = None
        if self.max_grad_norm > 0:
            grads = [p.grad for p in self.params if p.grad is not None]
            norm = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float()) for g in grads]))
            clip = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0).reshape(1).float()
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            if p.is_cuda:
                _bind()
                g = p.grad.contiguous()
                assert g.dtype in (torch.float32, torch.bfloat16)
                shadow = p.data_ptr() if p.dtype == torch.bfloat16 else None
                rc = _native.lib().idrak_adam8_step(
                    self.master[i].data_ptr(), shadow, g.data_ptr(), int(g.dtype == torch.bfloat16),
                    self.m8[i].data_ptr(), self.v8[i].data_ptr(), self.m_absmax[i].data_ptr(),
                    self.v_absmax[i].data_ptr(), p.numel(), self.lr, b1, b2, self.eps, bc1, bc2, self._wd[i], 1.0,
                    clip.data_ptr() if clip is not None else None, stream_ptr())
                _native.check(rc, "idrak_adam8_step")
            else:
                self._step_reference(i, p, bc1, bc2, clip)

    def _step_reference(self, i, p, bc1, bc2, clip):
        b1, b2 = self.betas
        n = p.numel()
        blocks = (n + BLOCK - 1) // BLOCK
        pad = blocks * BLOCK - n

        def blocked(t):
            return torch.nn.functional.pad(t.reshape(-1), (0, pad)).view(blocks, BLOCK)

        g = p.grad.reshape(-1).float() * (float(clip) if clip is not None else 1.0)
        m = blocked(signed_value(self.m8[i])) * self.m_absmax[i][:, None]
        v = blocked(unsigned_value(self.v8[i])) * self.v_absmax[i][:, None]
        gb = blocked(g)
        m = b1 * m + (1 - b1) * gb
        v = b2 * v + (1 - b2) * gb * gb
        w = blocked(self.master[i].reshape(-1))
        w = w * (1 - self.lr * self._wd[i]) - self.lr * (m / bc1) / (torch.sqrt(v / bc2) + self.eps)
        if pad:
            m.view(-1)[n:] = 0
            v.view(-1)[n:] = 0
        am, av = m.abs().amax(1), v.amax(1)
        self.m_absmax[i].copy_(am)
        self.v_absmax[i].copy_(av)
        self.m8[i].copy_(signed_code(torch.where(am[:, None] > 0, m / am[:, None].clamp_min(1e-38), torch.zeros_like(m))).view(-1)[:n])
        self.v8[i].copy_(unsigned_code(torch.where(av[:, None] > 0, v / av[:, None].clamp_min(1e-38), torch.zeros_like(v))).view(-1)[:n])
        self.master[i].reshape(-1).copy_(w.view(-1)[:n])
        if self.master[i].data_ptr() != p.data_ptr():
            p.copy_(self.master[i].to(p.dtype))

    def state_dict(self) -> dict:
        out = {"step": torch.tensor(float(self.step_count))}
        for i in range(len(self.params)):
            out[f"m8.{i}"], out[f"v8.{i}"] = self.m8[i].cpu(), self.v8[i].cpu()
            out[f"m_absmax.{i}"], out[f"v_absmax.{i}"] = self.m_absmax[i].cpu(), self.v_absmax[i].cpu()
        return out

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(float(state["step"]))
        for i in range(len(self.params)):
            for name, dst in (("m8", self.m8), ("v8", self.v8), ("m_absmax", self.m_absmax), ("v_absmax", self.v_absmax)):
                dst[i].copy_(state[f"{name}.{i}"])
