"""Packed weights: int8 (per output column) and int4 (groups of 32 input rows per column), and the
de-quant-fused linear op over them.

A packed weight describes ``W`` with rows = inputs and columns = outputs (the reference's ``[in, out]``
orientation):

* ``Int8Weight``: symmetric, ``scale[j] = max_i |w[i, j]| / 127``, one signed byte per value, rows padded
  to a multiple of four columns (four bytes per 32-bit word along each row).
* ``Int4Weight``: ``GroupSize = 32`` input rows of one column share a scale; nibble ``c`` of word ``w`` in
  row ``r`` is column ``8w + c``, two's complement in ``-8..7``; ``scales`` is
  ``[ceil(rows / 32), 8 * ceil(columns / 8)]``. The quantiser searches, per (group, column), 21 divisors
  around the extreme value and keeps the least-squares scale with the smallest squared error; a
  non-finite group gets scale 0 and zero nibbles.

Scales are kept in fp16 on the device (fp32 at the ``.ikw`` boundary, as the reference stores them).

``qlinear(x, weight)`` runs ``x @ W`` on the tcgen05 de-quantising GEMM; its backward pass returns
``dy @ W^T`` from the same kernel reading the codes transposed (the base is frozen: no weight
gradient). CPU tensors take the de-quantised matrix in plain PyTorch.

Reference: Int8Weight / Int4Weight (src/Idrak.Abstraction/Generation/Quantization.cs:382-470,659-1090),
ModuleExtensions.QuantizeInt8/Int4 (src/Idrak/Layers/ModuleExtensions.cs).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from ..ops._util import ptr, scratch, stream_ptr
from ..ops.gemm import _ACT_IDS, ACT_GELU

GROUP_SIZE = 32
PACKING_VERSION = 1

_BOUND = False


def _bind():
    """Declare the C signatures of the packed-weight entry points (once)."""
    global _BOUND
    if _BOUND:
        return
    import ctypes as C
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    _native.bind("idrak_qgemm", i, [vp, i, vp, vp, i, i, i, i, i, i, vp, i, i, i, vp, vp, i, i, vp, i, i, f, i, vp, vp])
    _native.bind("idrak_qdequant", i, [vp, vp, i, i, i, i, i, vp, i, vp])
    _BOUND = True


class Int8Weight:
    bits = 8

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, rows: int, cols: int):
        self.codes, self.scales, self.rows, self.cols = codes, scales, rows, cols    # codes [rows, ld] int8

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Int8Weight":
        """``w`` is ``[rows = in, cols = out]``."""
        wf = w.detach().float()
        rows, cols = wf.shape
        amax = wf.abs().amax(dim=0)
        scale = amax / 127.0
        safe = torch.where(scale > 0, scale, torch.ones_like(scale))
        q = torch.clamp(torch.round(wf / safe), -127, 127).to(torch.int8)
        ld = (cols + 7) // 8 * 8
        codes = torch.zeros((rows, ld), dtype=torch.int8, device=w.device)
        codes[:, :cols] = q
        return cls(codes.contiguous(), scale.to(torch.float16).contiguous(), rows, cols)

    def dequantize(self) -> torch.Tensor:
        return self.codes[:, : self.cols].float() * self.scales.float()[None, :]

    def to(self, device) -> "Int8Weight":
        return Int8Weight(self.codes.to(device), self.scales.to(device), self.rows, self.cols)

    def kmajor(self) -> torch.Tensor:
        """The codes transposed to ``[out, in]`` with the input index contiguous (rows padded to 16 bytes): what the
        few-row decode kernel streams. Made on first use and kept (it doubles the weight's code bytes)."""
        t = getattr(self, "_kmajor", None)
        if t is None or t.device != self.codes.device:
            kp = (self.rows + 15) // 16 * 16
            t = torch.zeros((self.cols, kp), dtype=torch.int8, device=self.codes.device)
            t[:, : self.rows] = self.codes[:, : self.cols].t()
            self._kmajor = t
        return t

    @property
    def ld(self) -> int:
        return self.codes.stride(0)

    @property
    def scale_ld(self) -> int:
        return self.scales.numel()

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel() * 2

    # .ikw buffers: packed bytes viewed as float32-typed words, scales as float32
    def buffers(self):
        words = self.codes[:, : (self.cols + 3) // 4 * 4].contiguous()
        if words.shape[1] % 4:
            pad = torch.zeros((self.rows, 4 - words.shape[1] % 4), dtype=torch.int8, device=words.device)
            words = torch.cat([words, pad], 1)
        return [words.contiguous().view(torch.float32), self.scales.float()]


class Int4Weight:
    bits = 4

    def __init__(self, words: torch.Tensor, scales: torch.Tensor, rows: int, cols: int):
        self.codes, self.scales, self.rows, self.cols = words, scales, rows, cols     # words [rows, cols8/8] int32

    @classmethod
    def quantize(cls, w: torch.Tensor, search: bool = True) -> "Int4Weight":
        wf = w.detach().float()
        rows, cols = wf.shape
        groups = (rows + GROUP_SIZE - 1) // GROUP_SIZE
        pad_rows = groups * GROUP_SIZE
        cols8 = (cols + 7) // 8 * 8
        wp = torch.zeros((pad_rows, cols8), dtype=torch.float32, device=w.device)
        wp[:rows, :cols] = wf
        g = wp.reshape(groups, GROUP_SIZE, cols8)
        finite = torch.isfinite(g).all(dim=1)
        g = torch.where(finite[:, None, :], g, torch.zeros_like(g))
        idx = g.abs().argmax(dim=1, keepdim=True)
        extreme = torch.gather(g, 1, idx)                       # signed value of largest magnitude [G,1,C]
        best_err = torch.full((groups, cols8), float("inf"), device=w.device)
        best_q = torch.zeros_like(g)
        best_d = torch.zeros((groups, cols8), device=w.device)
        steps = range(-10, 11) if search else (0,)
        nz = extreme != 0
        for step in steps:
            t = -8.0 + 0.1 * step
            inv = torch.where(nz, t / torch.where(nz, extreme, torch.ones_like(extreme)), torch.zeros_like(extreme))
            q = torch.clamp(torch.round(g * inv), -8, 7)
            qq = (q * q).sum(1)
            d = torch.where(qq > 0, (g * q).sum(1) / torch.where(qq > 0, qq, torch.ones_like(qq)),
                            torch.zeros_like(qq))
            err = ((g - q * d[:, None, :]) ** 2).sum(1)
            better = err < best_err
            best_err = torch.where(better, err, best_err)
            best_d = torch.where(better, d, best_d)
            best_q = torch.where(better[:, None, :], q, best_q)
        best_d = torch.where(finite, best_d, torch.zeros_like(best_d))
        q = best_q.reshape(pad_rows, cols8)[:rows].to(torch.int32) & 0xF
        q = q.reshape(rows, cols8 // 8, 8)
        shifts = torch.arange(8, device=w.device, dtype=torch.int32) * 4
        words = (q << shifts).sum(-1, dtype=torch.int64)
        words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
        return cls(words.contiguous(), best_d.to(torch.float16).contiguous(), rows, cols)

    def dequantize(self) -> torch.Tensor:
        w = self.codes.to(torch.int64) & 0xFFFFFFFF
        shifts = torch.arange(8, device=w.device, dtype=torch.int64) * 4
        nib = (w[:, :, None] >> shifts) & 0xF
        nib = torch.where(nib >= 8, nib - 16, nib).reshape(self.rows, -1).float()
        sc = self.scales.float().repeat_interleave(GROUP_SIZE, dim=0)[: self.rows]
        return (nib * sc)[:, : self.cols]

    def to(self, device) -> "Int4Weight":
        return Int4Weight(self.codes.to(device), self.scales.to(device), self.rows, self.cols)

    @property
    def ld(self) -> int:
        return self.codes.stride(0)

    @property
    def scale_ld(self) -> int:
        return self.scales.stride(0)

    def nbytes(self) -> int:
        return self.codes.numel() * 4 + self.scales.numel() * 2

    def buffers(self):
        return [self.codes.contiguous().view(torch.float32), self.scales.float()]


class Fp8Weight:
    """A frozen weight held as e4m3 codes ``[out, in]`` (K-major, what the fp8 tensor-core product reads) with one fp32
    scale per output unit. ``rows`` / ``cols`` follow the packed weights' ``[in, out]`` orientation. The forward product
    quantises the activations per row and runs on the ``kind::f8f6f4`` GEMM; the input gradient multiplies by the
    weight unpacked to bf16 (the gradient itself is not rounded to 8 bits)."""
    bits = 8
    kind = "fp8"

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, rows: int, cols: int):
        self.codes, self.scales, self.rows, self.cols = codes, scales, rows, cols      # codes [cols = out, rows = in]

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Fp8Weight":
        """``w`` is ``[rows = in, cols = out]``."""
        from ..ops.gemm8 import quantize_rows
        rows, cols = w.shape
        q = quantize_rows(w.detach().t().contiguous().to(torch.bfloat16))
        return cls(q.codes, q.scales, rows, cols)

    def as_rows(self):
        from ..ops.gemm8 import Float8Rows
        return Float8Rows(self.codes, self.scales)

    def dense_out_in(self) -> torch.Tensor:
        """The weight as bf16 ``[out, in]``."""
        return self.as_rows().dequantize(torch.bfloat16)

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[in, out]`` like the other packed weights."""
        return self.as_rows().dequantize(torch.float32).t()

    def to(self, device) -> "Fp8Weight":
        return Fp8Weight(self.codes.to(device), self.scales.to(device), self.rows, self.cols)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel() * 4

    def buffers(self):
        return [self.codes, self.scales]


def quantize_weight(w_in_out: torch.Tensor, kind: str):
    if kind == "int8":
        return Int8Weight.quantize(w_in_out)
    if kind == "int4":
        return Int4Weight.quantize(w_in_out)
    if kind == "fp8":
        return Fp8Weight.quantize(w_in_out)
    raise ValueError(f"unknown packed format '{kind}' (int8, int4, fp8)")


def _fp8_product(x2, w: "Fp8Weight", transposed, bias, residual, act, out):
    from ..ops.gemm import gemm
    from ..ops.gemm8 import gemm8, quantize_rows
    if act is not None:
        raise ValueError("the fp8 base has no fused activation epilogue")
    if transposed:                                   # dy [M, out] -> dx [M, in]
        return gemm(x2, w.dense_out_in(), b_mn=True, bias=bias, residual=residual, out=out)
    if x2.is_cuda and w.rows % 16 == 0:
        y = gemm8(quantize_rows(x2.to(torch.bfloat16)), w.as_rows(), bias, out=out)
        if residual is not None:
            y += residual
        return y
    return gemm(x2, w.dense_out_in(), bias=bias, residual=residual, out=out)


# --------------------------------------------------------------------------- the op
FEW_ROW_INT8_KERNEL = True   # int8 weights, few rows: the few-row kernel that reads the codes directly (csrc/skinny8_gemm.cu)
FEW_ROWS = 64           # up to this many rows (decode steps) the weight is unpacked first as well: see qgemm
DENSE_ROWS = 512        # from this many activation rows on, the weight is unpacked to bf16 first and multiplied densely


def qgemm(x2: torch.Tensor, w, transposed: bool = False, bias=None, residual=None, act: Optional[str] = None,
          out: Optional[torch.Tensor] = None, splits: Optional[int] = None):
    """``x2 @ W`` (or ``x2 @ W^T``) with the fused epilogue of the dense GEMM."""
    M = x2.shape[0]
    N = w.rows if transposed else w.cols
    K = w.cols if transposed else w.rows
    assert x2.shape[1] == K and x2.stride(1) == 1
    if isinstance(w, Fp8Weight):
        return _fp8_product(x2, w, transposed, bias, residual, act, out)
    if not x2.is_cuda:
        wf = w.dequantize()
        y = x2.float() @ (wf.t() if transposed else wf)
        if bias is not None:
            y = y + bias.float()
        aux = None
        if _ACT_IDS[act] == ACT_GELU:
            aux = y.to(x2.dtype)
            y = torch.nn.functional.gelu(aux.float(), approximate="tanh")
        if residual is not None:
            y = y + residual.float()
        y = y.to(x2.dtype)
        return (y, aux) if aux is not None else y
    if (M <= FEW_ROWS and isinstance(w, Int8Weight) and not transposed and act is None and x2.is_cuda
            and x2.dtype == torch.bfloat16 and K % 16 == 0 and x2.stride(0) % 8 == 0 and FEW_ROW_INT8_KERNEL
            and _native.has("idrak_skinny8_gemm")):
        # decode steps over int8 weights: the codes are streamed once (half the bytes of bf16) and expanded to bf16
        # operand tiles inside the few-row kernel
        from ..ops.skinny import skinny8_linear
        return skinny8_linear(x2, w, bias, residual, out=out)
    if ((M >= DENSE_ROWS or M <= FEW_ROWS) and x2.dtype == torch.bfloat16 and w.cols % 8 == 0
            and x2.stride(0) % 8 == 0):
        # many rows: unpacking the weight once (a bandwidth-bound pass over it) and running the dense tensor-core GEMM
        # beats unpacking inside the GEMM's producer warps. Few rows (decoding): the same holds, measured at 64 rows of
        # a 4096 x 4096 int8 weight 81 us in the unpacking GEMM against 13 us to unpack (the bf16 copy of one
        # projection stays in L2) plus 17 us for the split-K product over it
        from ..ops.gemm import gemm
        return gemm(x2, dequantize_bf16(w), b_mn=not transposed, bias=bias, residual=residual, act=act, out=out)
    _bind()
    lib = _native.lib()
    fn = lib.idrak_qgemm
    if out is None:
        out = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
    aux_t = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device) if _ACT_IDS[act] == ACT_GELU else None
    if splits is None:
        splits = lib.idrak_gemm_pick_splits(M, N, K, 128 if N <= 128 else 256)
    ws = scratch("qgemm_splitk", splits * M * N, torch.float32, x2.device) if splits > 1 else None
    rc = fn(x2.data_ptr(), x2.stride(0), w.codes.data_ptr(), w.scales.data_ptr(), w.rows, w.cols, w.ld, w.scale_ld,
            w.bits, int(transposed), out.data_ptr(), out.stride(0), 0, M, ptr(bias), ptr(residual),
            residual.stride(0) if residual is not None else 0, _ACT_IDS[act], ptr(aux_t),
            aux_t.stride(0) if aux_t is not None else 0, 0, 1.0, int(splits), ptr(ws), stream_ptr())
    _native.check(rc, "idrak_qgemm")
    return (out, aux_t) if aux_t is not None else out


def dequantize_bf16(w) -> torch.Tensor:
    """The packed weight as a bf16 ``[rows, cols]`` matrix (GPU kernel when on the device)."""
    if isinstance(w, Fp8Weight):
        return w.dense_out_in().t().contiguous()
    if not w.codes.is_cuda:
        return w.dequantize().to(torch.bfloat16)
    _bind()
    out = torch.empty((w.rows, w.cols), dtype=torch.bfloat16, device=w.codes.device)
    rc = _native.lib().idrak_qdequant(w.codes.data_ptr(), w.scales.data_ptr(), w.rows, w.cols, w.ld, w.scale_ld,
                                      w.bits, out.data_ptr(), out.stride(0), stream_ptr())
    _native.check(rc, "idrak_qdequant")
    return out


class _QLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        r2 = residual.reshape(-1, w.cols) if residual is not None else None
        y = qgemm(x2, w, False, bias, r2)
        ctx.w = w
        ctx.flags = (bias is not None, residual is not None)
        return y.reshape(*shape[:-1], w.cols)

    @staticmethod
    def backward(ctx, dy):
        w = ctx.w
        dy2 = dy.reshape(-1, w.cols)
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        dx = qgemm(dy2, w, True).reshape(*dy.shape[:-1], w.rows) if ctx.needs_input_grad[0] else None
        db = None
        if ctx.flags[0] and ctx.needs_input_grad[2]:
            from ..ops.rowops import colsum
            db = colsum(dy2)
        return dx, None, db, (dy if ctx.flags[1] else None)


class _QLowRankLinear(torch.autograd.Function):
    """``y = x W + (x A^T) B^T (+ b) (+ residual)`` over a packed ``W`` ``[in, out]`` for many rows: the weight is unpacked
    once per pass and the low-rank term rides in the same tcgen05 product as one more block of K."""

    @staticmethod
    def forward(ctx, x, w, bias, residual, A, B):
        from ..ops.gemm import gemm, gemm_lowrank
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        r2 = residual.reshape(-1, w.cols) if residual is not None else None
        t = gemm(x2, A)                                                              # [M, R]
        y = gemm_lowrank(x2, dequantize_bf16(w), t, B.t().contiguous(), b_mn=True, bias=bias, residual=r2)
        ctx.w = w
        ctx.save_for_backward(x2, A, B, t)
        ctx.flags = (bias is not None, residual is not None)
        return y.reshape(*shape[:-1], w.cols)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm, gemm_lowrank
        w = ctx.w
        x2, A, B, t = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.cols)
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        dt = gemm(dy2, B, b_mn=True)                                                 # [M, R]
        dx = db = dA = dB = None
        if ctx.needs_input_grad[0]:
            dx = gemm_lowrank(dy2, dequantize_bf16(w), dt, A.t().contiguous()).reshape(*dy.shape[:-1], w.rows)
        if ctx.flags[0] and ctx.needs_input_grad[2]:
            from ..ops.rowops import colsum
            db = colsum(dy2)
        if ctx.needs_input_grad[4]:
            dA = gemm(dt, x2, a_mn=True, b_mn=True)
        if ctx.needs_input_grad[5]:
            dB = gemm(dy2, t, a_mn=True, b_mn=True)
        return dx, None, db, (dy if ctx.flags[1] else None), dA, dB


def qlowrank_linear(x, w, bias, residual, A, B):
    """``qlinear`` plus the stacked adapters ``A`` ``[R, in]`` / ``B`` ``[out, R]``; the fused kernel for bf16 inputs of
    ``DENSE_ROWS`` rows or more, separate products otherwise."""
    from ..ops.gemm import lowrank_supported
    rows = x.numel() // x.shape[-1]
    if (lowrank_supported(x, A.shape[0]) and rows >= DENSE_ROWS and w.cols % 8 == 0 and w.rows % 8 == 0
            and w.codes.is_cuda and not isinstance(w, Fp8Weight)):
        return _QLowRankLinear.apply(x, w, bias, residual, A, B)
    from ..ops import linear
    return qlinear(x, w, bias, residual) + linear(linear(x, A), B)


def qlinear(x: torch.Tensor, w, bias: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W + bias (+ residual)`` over a packed weight ``W`` ``[in, out]``."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _QLinear.apply(x, w, bias, residual)
    y = (x.float() @ w.dequantize().to(x.device)).to(x.dtype)
    if bias is not None:
        y = y + bias
    return y + residual if residual is not None else y
