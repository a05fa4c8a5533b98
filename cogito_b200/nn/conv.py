"""Conv2d (im2col + tensor-core GEMM), MaxPool2d and BatchNorm over [N, C, H, W] / [N, F].

Reference: Conv2D is im2col + naive GEMM with weights [out_c, in_c*k*k] and Kaiming-normal
init (src/layers/conv2d.c:23-421); MaxPool2D keeps arg-max indices (``:249-421``); batch norm
uses ``running = momentum * running + (1 - momentum) * batch`` with biased variance
(src/layers/activations.c:496-499,618-619).  On CUDA the unfold / fold / pooling / statistics
run in the library's kernels and the contraction in the tcgen05 GEMM; on CPU the same maths
goes through PyTorch ops.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import _lib
from ..ops.gemm import gemm
from ..utils import rng


def _out_hw(H, W, k, stride, pad):
    return (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1


class _Conv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, k, stride, pad):
        N, C, H, W = x.shape
        OC = weight.shape[0]
        OH, OW = _out_hw(H, W, k, stride, pad)
        CK = C * k * k
        ld = (CK + 7) // 8 * 8                                   # TMA rows must be 16-byte multiples
        xb = x.to(torch.bfloat16).contiguous()
        col = torch.zeros(N * OH * OW, ld, dtype=torch.bfloat16, device=x.device)
        L = _lib.lib()
        _lib.check(L.cgk_im2col(1, xb.data_ptr(), col.data_ptr(), N, C, H, W, k, stride, pad, OH, OW, ld, _lib.stream_ptr()), "cgk_im2col")
        _lib.count_launch()
        wp = torch.zeros(OC, ld, dtype=torch.bfloat16, device=x.device)
        wp[:, :CK] = weight.to(torch.bfloat16)
        y = gemm(col, wp, bias=None if bias is None else bias.to(torch.bfloat16), out_dtype=torch.float32)   # [N*OH*OW, OC]
        ctx.save_for_backward(col, wp, weight, bias if bias is not None else torch.empty(0))
        ctx.geom = (N, C, H, W, k, stride, pad, OH, OW, CK, ld)
        return y.view(N, OH, OW, OC).permute(0, 3, 1, 2).contiguous().to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        col, wp, weight, bias = ctx.saved_tensors
        N, C, H, W, k, stride, pad, OH, OW, CK, ld = ctx.geom
        OC = wp.shape[0]
        g = dy.permute(0, 2, 3, 1).reshape(N * OH * OW, OC).to(torch.bfloat16).contiguous()
        dw = gemm(g, col, a_mn=True, b_mn=True, out_dtype=torch.float32)[:, :CK]          # G^T col
        dcol = gemm(g, wp, b_mn=True)                                                      # G W  [rows, ld]
        dx = torch.zeros(N, C, H, W, dtype=torch.float32, device=dy.device)
        _lib.check(_lib.lib().cgk_col2im(1, dcol.data_ptr(), dx.data_ptr(), N, C, H, W, k, stride, pad, OH, OW, ld,
                                         _lib.stream_ptr()), "cgk_col2im")
        _lib.count_launch()
        db = g.float().sum(0).to(bias.dtype) if bias.numel() else None
        return dx.to(dy.dtype), dw.to(weight.dtype).view_as(weight), db, None, None, None


class Conv2d(nn.Module):
    """Square kernel, equal stride and padding on both axes; weight [out_c, in_c * k * k]."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True, device=None, dtype=None):
        super().__init__()
        self.in_channels, self.out_channels, self.k, self.stride, self.padding = in_channels, out_channels, kernel_size, stride, padding
        fan_in = in_channels * kernel_size * kernel_size
        w = torch.empty(out_channels, fan_in, device=device, dtype=dtype)
        self.weight = nn.Parameter(rng.normal_(w, math.sqrt(2.0 / fan_in), rng.layer_generator()))
        self.bias = nn.Parameter(torch.zeros(out_channels, device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        if x.is_cuda:
            return _Conv2dFn.apply(x, self.weight, self.bias, self.k, self.stride, self.padding)
        w = self.weight.view(self.out_channels, self.in_channels, self.k, self.k)
        return torch.nn.functional.conv2d(x, w, self.bias, self.stride, self.padding)


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, stride):
        N, C, H, W = x.shape
        OH, OW = _out_hw(H, W, k, stride, 0)
        xf = x.float().contiguous()
        y = torch.empty(N, C, OH, OW, dtype=torch.float32, device=x.device)
        arg = torch.empty(N, C, OH, OW, dtype=torch.int32, device=x.device)
        _lib.check(_lib.lib().cgk_maxpool_forward(xf.data_ptr(), y.data_ptr(), arg.data_ptr(), N, C, H, W, k, stride, OH, OW,
                                                  _lib.stream_ptr()), "cgk_maxpool_forward")
        _lib.count_launch()
        ctx.save_for_backward(arg)
        ctx.geom = (N, C, H, W, OH, OW)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (arg,) = ctx.saved_tensors
        N, C, H, W, OH, OW = ctx.geom
        dx = torch.zeros(N, C, H, W, dtype=torch.float32, device=dy.device)
        g = dy.float().contiguous()
        _lib.check(_lib.lib().cgk_maxpool_backward(g.data_ptr(), arg.data_ptr(), dx.data_ptr(), N, C, H, W, OH, OW,
                                                   _lib.stream_ptr()), "cgk_maxpool_backward")
        _lib.count_launch()
        return dx.to(dy.dtype), None, None


class MaxPool2d(nn.Module):
    def __init__(self, kernel_size, stride=None):
        super().__init__()
        self.k, self.stride = kernel_size, stride or kernel_size

    def forward(self, x):
        if x.is_cuda:
            return _MaxPoolFn.apply(x, self.k, self.stride)
        return torch.nn.functional.max_pool2d(x, self.k, self.stride)


class _BatchNormFn(torch.autograd.Function):
    """x [B, F] fp32 on the kernels (one CTA per feature)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, eps, momentum, training):
        B, F = x.shape
        xf = x.float().contiguous()
        y = torch.empty_like(xf)
        mean, rstd = torch.empty(F, device=x.device), torch.empty(F, device=x.device)
        # the kernels read fp32 scale and shift; a flat bf16 optimizer buffer may hold them in bf16
        ctx.param_dtype = gamma.dtype
        gamma, beta = gamma.float().contiguous(), beta.float().contiguous()
        _lib.check(_lib.lib().cgk_batchnorm_forward(xf.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
                                                    running_mean.data_ptr(), running_var.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                                    B, F, eps, momentum, int(training), _lib.stream_ptr()), "cgk_batchnorm_forward")
        _lib.count_launch()
        ctx.save_for_backward(xf, gamma, mean, rstd)
        ctx.training = training
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xf, gamma, mean, rstd = ctx.saved_tensors
        if not ctx.training:
            return (dy.float() * gamma * rstd).to(dy.dtype), None, None, None, None, None, None, None
        B, F = xf.shape
        g = dy.float().contiguous()
        dx, dgamma, dbeta = torch.empty_like(xf), torch.empty(F, device=g.device), torch.empty(F, device=g.device)
        _lib.check(_lib.lib().cgk_batchnorm_backward(xf.data_ptr(), g.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                                     dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), B, F, _lib.stream_ptr()),
                   "cgk_batchnorm_backward")
        _lib.count_launch()
        return dx.to(dy.dtype), dgamma.to(ctx.param_dtype), dbeta.to(ctx.param_dtype), None, None, None, None, None


class BatchNorm(nn.Module):
    """Batch normalisation over [B, F] or per channel of [N, C, H, W] (fp32 parameters)."""

    def __init__(self, features, eps=1e-5, momentum=0.1, device=None):
        super().__init__()
        self.eps, self.momentum = eps, momentum
        self.weight = nn.Parameter(torch.ones(features, device=device))
        self.bias = nn.Parameter(torch.zeros(features, device=device))
        self.register_buffer("running_mean", torch.zeros(features, device=device))
        self.register_buffer("running_var", torch.ones(features, device=device))

    def forward(self, x):
        four_d = x.dim() == 4
        if four_d:
            N, C, H, W = x.shape
            x2 = x.permute(0, 2, 3, 1).reshape(-1, C)
        else:
            x2 = x
        if x2.is_cuda:
            y = _BatchNormFn.apply(x2, self.weight, self.bias, self.running_mean, self.running_var, self.eps, self.momentum, self.training)
        else:
            xf = x2.float()
            if self.training:
                mean, var = xf.mean(0), xf.var(0, unbiased=False)
                with torch.no_grad():
                    self.running_mean.mul_(self.momentum).add_((1 - self.momentum) * mean)
                    self.running_var.mul_(self.momentum).add_((1 - self.momentum) * var)
            else:
                mean, var = self.running_mean, self.running_var
            y = ((xf - mean) * torch.rsqrt(var + self.eps) * self.weight + self.bias).to(x.dtype)
        return y.view(N, H, W, C).permute(0, 3, 1, 2).contiguous() if four_d else y
