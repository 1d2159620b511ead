"""Convolution and pooling on the device: dense convolution as patch rows around the tcgen05 GEMM, depthwise
convolution, max and average pooling, each with its backward pass (``csrc/conv.cu``). N x C x H x W tensors.

bf16 CUDA tensors take the kernels for everything; fp32 CUDA tensors take them for pooling and depthwise convolution
(exact in fp32) while a dense fp32 convolution stays with the library unless ``allow_bf16_products`` is set, because its
products here round the operands to bf16 (fp32 accumulation). CPU tensors run the PyTorch statements.

Reference: Tensor.Convolution / MaxPool / AvgPool (src/Idrak.Abstraction/Tensors/Tensor.Convolution.cs), conv_fwd /
conv_bwd_input / conv_bwd_weight / conv_dw / avgpool / im2col / col2im / maxpool
(src/Idrak.Gpu/Cuda/PtxKernels.Convolution.cs, PtxKernels.Advanced.cs:12).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from .. import _native
from ._util import ptr, stream_ptr

_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def _pair(v):
    return (int(v[0]), int(v[1])) if isinstance(v, (tuple, list)) else (int(v), int(v))


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


def _out_size(size, k, s, p, d=1, ceil_mode=False):
    span = size + 2 * p - d * (k - 1) - 1
    if ceil_mode:
        o = -(-span // s) + 1
        if (o - 1) * s >= size + p:          # the last window must start inside the input or its left padding
            o -= 1
        return o
    return span // s + 1


def _shape(N, Cc, H, W, KH, KW, OH, OW, stride, padding, dilation):
    return (C.c_int * 14)(N, Cc, H, W, KH, KW, OH, OW, stride[0], stride[1], padding[0], padding[1], dilation[0],
                          dilation[1])


def _round8(n):
    return (n + 7) // 8 * 8


# ---------------------------------------------------------------------------------------------------- dense convolution
class _Conv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation):
        from .gemm import gemm
        lib = _native.lib()
        N, Cc, H, W = x.shape
        OC, _, KH, KW = weight.shape
        OH = _out_size(H, KH, stride[0], padding[0], dilation[0])
        OW = _out_size(W, KW, stride[1], padding[1], dilation[1])
        K, Kp, OCp = Cc * KH * KW, _round8(Cc * KH * KW), _round8(OC)
        shape = _shape(N, Cc, H, W, KH, KW, OH, OW, stride, padding, dilation)
        dt = _DTYPES[x.dtype]
        rows = torch.empty((N * OH * OW, Kp), dtype=torch.bfloat16, device=x.device)
        _native.check(lib.idrak_im2col(dt, x.data_ptr(), rows.data_ptr(), shape, Kp, stream_ptr()), "idrak_im2col")
        wmat = torch.zeros((OCp, Kp), dtype=torch.bfloat16, device=x.device)
        wmat[:OC, :K] = weight.reshape(OC, K)
        out_rows = gemm(rows, wmat)                                        # [N*OH*OW, OCp]
        y = torch.empty((N, OC, OH, OW), dtype=x.dtype, device=x.device)
        b32 = None if bias is None else bias.float().contiguous()
        _native.check(lib.idrak_rows_to_nchw(dt, out_rows.data_ptr(), y.data_ptr(), ptr(b32), N, OC, OH * OW, OCp,
                                             stream_ptr()), "idrak_rows_to_nchw")
        ctx.save_for_backward(rows, wmat)
        ctx.spec = (tuple(x.shape), tuple(weight.shape), bias is not None, stride, padding, dilation, OH, OW, x.dtype,
                    weight.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .gemm import gemm
        from .reduce import sum_axis
        lib = _native.lib()
        rows, wmat = ctx.saved_tensors
        (N, Cc, H, W), (OC, _, KH, KW), has_bias, stride, padding, dilation, OH, OW, xdt, wdt, bdt = ctx.spec
        K, Kp, OCp = Cc * KH * KW, rows.shape[1], wmat.shape[0]
        dy = _c(dy)
        dt = _DTYPES[dy.dtype]
        shape = _shape(N, Cc, H, W, KH, KW, OH, OW, stride, padding, dilation)
        dy_rows = torch.empty((N * OH * OW, OCp), dtype=torch.bfloat16, device=dy.device)
        _native.check(lib.idrak_nchw_to_rows(dt, dy.data_ptr(), dy_rows.data_ptr(), N, OC, OH * OW, OCp, stream_ptr()),
                      "idrak_nchw_to_rows")
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            drows = gemm(dy_rows, wmat, b_mn=True)                         # [M, OCp] x [OCp, Kp]
            dx = torch.empty((N, Cc, H, W), dtype=xdt, device=dy.device)
            _native.check(lib.idrak_col2im(_DTYPES[xdt], drows.data_ptr(), dx.data_ptr(), shape, Kp, 0, stream_ptr()),
                          "idrak_col2im")
        if ctx.needs_input_grad[1]:
            dwm = gemm(dy_rows, rows, a_mn=True, b_mn=True, out_dtype=torch.float32)   # [OCp, Kp]
            dw = dwm[:OC, :K].reshape(OC, Cc, KH, KW).to(wdt)
        if has_bias and ctx.needs_input_grad[2]:
            db = sum_axis(dy_rows, 0)[:OC].to(bdt)
        return dx, dw, db, None, None, None


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups: int = 1, allow_bf16_products: bool = False):
    """2-D convolution (cross-correlation, like ``torch.nn.functional.conv2d``)."""
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    depthwise = groups > 1 and groups == x.shape[1] and weight.shape[0] == groups and weight.shape[1] == 1
    on_device = x.is_cuda and x.dtype in _DTYPES and x.numel() > 0
    if on_device and depthwise:
        return depthwise_conv2d(x, weight, bias, stride, padding, dilation)
    dense_ok = on_device and groups == 1 and (x.dtype == torch.bfloat16 or allow_bf16_products)
    if not dense_ok:
        return F.conv2d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), stride, padding, dilation,
                        groups)
    return _Conv2d.apply(_c(x), weight, bias, stride, padding, dilation)


def conv1d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups: int = 1, allow_bf16_products: bool = False):
    """1-D convolution over ``[N, C, L]`` as a 2-D one with a height of one."""
    y = conv2d(x.unsqueeze(2), weight.unsqueeze(2), bias, (1, int(stride)), (0, int(padding)), (1, int(dilation)),
               groups, allow_bf16_products)
    return y.squeeze(2)


# ------------------------------------------------------------------------------------------------------------ depthwise
class _Depthwise(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation):
        N, Cc, H, W = x.shape
        KH, KW = weight.shape[-2:]
        OH = _out_size(H, KH, stride[0], padding[0], dilation[0])
        OW = _out_size(W, KW, stride[1], padding[1], dilation[1])
        w = _c(weight.to(x.dtype).reshape(Cc, KH, KW))
        b = None if bias is None else _c(bias.to(x.dtype))
        y = torch.empty((N, Cc, OH, OW), dtype=x.dtype, device=x.device)
        shape = _shape(N, Cc, H, W, KH, KW, OH, OW, stride, padding, dilation)
        rc = _native.lib().idrak_dw_conv(_DTYPES[x.dtype], x.data_ptr(), w.data_ptr(), ptr(b), y.data_ptr(), shape,
                                         stream_ptr())
        _native.check(rc, "idrak_dw_conv")
        ctx.save_for_backward(x, w)
        ctx.spec = (stride, padding, dilation, OH, OW, tuple(weight.shape), weight.dtype,
                    None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        stride, padding, dilation, OH, OW, wshape, wdt, bdt = ctx.spec
        N, Cc, H, W = x.shape
        KH, KW = w.shape[-2:]
        dy = _c(dy)
        lib = _native.lib()
        dt = _DTYPES[x.dtype]
        shape = _shape(N, Cc, H, W, KH, KW, OH, OW, stride, padding, dilation)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _native.check(lib.idrak_dw_conv_bwd_input(dt, dy.data_ptr(), w.data_ptr(), dx.data_ptr(), shape,
                                                      stream_ptr()), "idrak_dw_conv_bwd_input")
        if ctx.needs_input_grad[1] or (bdt is not None and ctx.needs_input_grad[2]):
            dw32 = torch.empty((Cc, KH, KW), dtype=torch.float32, device=x.device)
            db32 = torch.empty(Cc, dtype=torch.float32, device=x.device) if bdt is not None else None
            _native.check(lib.idrak_dw_conv_bwd_weight(dt, x.data_ptr(), dy.data_ptr(), dw32.data_ptr(), ptr(db32),
                                                       shape, stream_ptr()), "idrak_dw_conv_bwd_weight")
            dw = dw32.reshape(wshape).to(wdt)
            db = None if db32 is None else db32.to(bdt)
        return dx, dw, db, None, None, None


def depthwise_conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1):
    """One filter per channel: ``weight`` ``[C, 1, KH, KW]``."""
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    if not (x.is_cuda and x.dtype in _DTYPES and x.numel() > 0):
        return F.conv2d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), stride, padding, dilation,
                        x.shape[1])
    return _Depthwise.apply(_c(x), weight, bias, stride, padding, dilation)


# -------------------------------------------------------------------------------------------------------------- pooling
class _MaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, padding, dilation, ceil_mode):
        N, Cc, H, W = x.shape
        OH = _out_size(H, kernel[0], stride[0], padding[0], dilation[0], ceil_mode)
        OW = _out_size(W, kernel[1], stride[1], padding[1], dilation[1], ceil_mode)
        y = torch.empty((N, Cc, OH, OW), dtype=x.dtype, device=x.device)
        index = torch.empty((N, Cc, OH, OW), dtype=torch.int32, device=x.device)
        shape = _shape(N, Cc, H, W, kernel[0], kernel[1], OH, OW, stride, padding, dilation)
        rc = _native.lib().idrak_maxpool(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), index.data_ptr(), shape,
                                         stream_ptr())
        _native.check(rc, "idrak_maxpool")
        ctx.save_for_backward(index)
        ctx.spec = (tuple(x.shape), kernel, stride, padding, dilation, OH, OW)
        return y

    @staticmethod
    def backward(ctx, dy):
        (index,) = ctx.saved_tensors
        (N, Cc, H, W), kernel, stride, padding, dilation, OH, OW = ctx.spec
        dy = _c(dy)
        dx = torch.empty((N, Cc, H, W), dtype=dy.dtype, device=dy.device)
        shape = _shape(N, Cc, H, W, kernel[0], kernel[1], OH, OW, stride, padding, dilation)
        rc = _native.lib().idrak_maxpool_bwd(_DTYPES[dy.dtype], dy.data_ptr(), index.data_ptr(), dx.data_ptr(), shape,
                                             stream_ptr())
        _native.check(rc, "idrak_maxpool_bwd")
        return dx, None, None, None, None, None


def max_pool2d(x, kernel, stride=None, padding=0, dilation=1, ceil_mode: bool = False):
    kernel = _pair(kernel)
    stride = kernel if stride is None else _pair(stride)
    padding, dilation = _pair(padding), _pair(dilation)
    if not (x.is_cuda and x.dtype in _DTYPES and x.dim() == 4 and x.numel() > 0):
        return F.max_pool2d(x, kernel, stride, padding, dilation, ceil_mode)
    return _MaxPool.apply(_c(x), kernel, stride, padding, dilation, bool(ceil_mode))


class _AvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, padding, ceil_mode, include_pad):
        N, Cc, H, W = x.shape
        OH = _out_size(H, kernel[0], stride[0], padding[0], 1, ceil_mode)
        OW = _out_size(W, kernel[1], stride[1], padding[1], 1, ceil_mode)
        y = torch.empty((N, Cc, OH, OW), dtype=x.dtype, device=x.device)
        shape = _shape(N, Cc, H, W, kernel[0], kernel[1], OH, OW, stride, padding, (1, 1))
        rc = _native.lib().idrak_avgpool(_DTYPES[x.dtype], x.data_ptr(), y.data_ptr(), shape, int(include_pad),
                                         stream_ptr())
        _native.check(rc, "idrak_avgpool")
        ctx.spec = (tuple(x.shape), kernel, stride, padding, include_pad, OH, OW)
        return y

    @staticmethod
    def backward(ctx, dy):
        (N, Cc, H, W), kernel, stride, padding, include_pad, OH, OW = ctx.spec
        dy = _c(dy)
        dx = torch.empty((N, Cc, H, W), dtype=dy.dtype, device=dy.device)
        shape = _shape(N, Cc, H, W, kernel[0], kernel[1], OH, OW, stride, padding, (1, 1))
        rc = _native.lib().idrak_avgpool_bwd(_DTYPES[dy.dtype], dy.data_ptr(), dx.data_ptr(), shape, int(include_pad),
                                             stream_ptr())
        _native.check(rc, "idrak_avgpool_bwd")
        return dx, None, None, None, None, None


def avg_pool2d(x, kernel, stride=None, padding=0, ceil_mode: bool = False, count_include_pad: bool = True):
    kernel = _pair(kernel)
    stride = kernel if stride is None else _pair(stride)
    padding = _pair(padding)
    # with ceil_mode a window may hang over the padded edge, where the divisor rule of the library differs: leave it there
    if ceil_mode or not (x.is_cuda and x.dtype in _DTYPES and x.dim() == 4 and x.numel() > 0):
        return F.avg_pool2d(x, kernel, stride, padding, ceil_mode, count_include_pad)
    return _AvgPool.apply(_c(x), kernel, stride, padding, False, bool(count_include_pad))
