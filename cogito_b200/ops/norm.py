"""LayerNorm / RMSNorm with the residual add fused into the forward kernel.

``layer_norm(x, gamma, beta, residual=r)`` returns ``(y, s)`` where ``s = x + r``
is the updated residual stream (written by the same kernel) and
``y = LN(s)``; without ``residual`` it returns ``y`` only.
Reference semantics: cg_cuda_layernorm_forward / cg_cuda_rmsnorm_forward
(src/cuda/tensor_kernels.c:812-909), rmsnorm_forward/backward
(src/layers/normalization.c:14-105): ``y = x * rsqrt(mean(x^2) + eps) * w``.
"""
from __future__ import annotations

import torch

from . import _lib

_BF16 = torch.bfloat16


def norm_forward_raw(x2, gamma, beta, eps, rms, residual2=None, want_sum=False):
    """x2: [rows, D] bf16.  Returns (y, sum_or_None, mean, rstd)."""
    rows, D = x2.shape
    if not x2.is_cuda:
        s = x2.float() + (residual2.float() if residual2 is not None else 0.0)
        if residual2 is not None:
            s = s.to(x2.dtype).float()
        if rms:
            mean = torch.zeros(rows)
            rstd = torch.rsqrt((s * s).mean(-1) + eps)
            y = s * rstd[:, None] * gamma.float()
        else:
            mean = s.mean(-1)
            var = ((s - mean[:, None]) ** 2).mean(-1)
            rstd = torch.rsqrt(var + eps)
            y = (s - mean[:, None]) * rstd[:, None] * gamma.float()
            if beta is not None:
                y = y + beta.float()
        return y.to(x2.dtype), (s.to(x2.dtype) if want_sum else None), mean, rstd
    if x2.dtype != _BF16:
        raise TypeError("norm: CUDA activations must be bf16")
    y = torch.empty_like(x2)
    s = torch.empty_like(x2) if (want_sum and residual2 is not None) else None
    mean = torch.empty(rows, device=x2.device, dtype=torch.float32)
    rstd = torch.empty(rows, device=x2.device, dtype=torch.float32)
    _lib.check(_lib.lib().cgk_norm_forward(
        x2.data_ptr(), _lib.ptr(residual2), gamma.data_ptr(), _lib.ptr(beta), y.data_ptr(), _lib.ptr(s),
        mean.data_ptr(), rstd.data_ptr(), rows, D, float(eps), int(rms), _lib.stream_ptr()), "cgk_norm_forward")
    _lib.count_launch()
    return y, s, mean, rstd


def norm_backward_raw(dy2, s2, gamma, mean, rstd, rms, dres2=None, dgamma_out=None, dbeta_out=None):
    """Returns (dx, dgamma fp32, dbeta fp32 or None).  When *_out are given the
    parameter gradients are accumulated into them."""
    rows, D = s2.shape
    if not s2.is_cuda:
        sf = s2.float()
        xh = sf * rstd[:, None] if rms else (sf - mean[:, None]) * rstd[:, None]
        gd = dy2.float() * gamma.float()
        s1 = 0.0 if rms else gd.mean(-1, keepdim=True)
        s2m = (gd * xh).mean(-1, keepdim=True)
        dx = rstd[:, None] * (gd - s1 - xh * s2m)
        if dres2 is not None:
            dx = dx + dres2.float()
        dg = (dy2.float() * xh).sum(0)
        db = dy2.float().sum(0)
        if dgamma_out is not None:
            dgamma_out += dg
            dg = dgamma_out
        if dbeta_out is not None:
            dbeta_out += db
            db = dbeta_out
        return dx.to(dy2.dtype), dg, (None if rms else db)
    L = _lib.lib()
    dx = torch.empty_like(s2)
    acc = dgamma_out is not None
    dg = dgamma_out if acc else torch.empty(D, device=s2.device, dtype=torch.float32)
    db = None
    if not rms:
        db = dbeta_out if dbeta_out is not None else torch.empty(D, device=s2.device, dtype=torch.float32)
        if acc and dbeta_out is None:
            db.zero_()
    scratch = torch.empty(max(1, L.cgk_norm_backward_scratch_elems(rows, D)), device=s2.device,
                          dtype=torch.float32)
    if dy2.stride(-1) != 1 or dy2.stride(0) != D:
        dy2 = dy2.contiguous()
    _lib.check(L.cgk_norm_backward(
        dy2.data_ptr(), s2.data_ptr(), gamma.data_ptr(), _lib.ptr(mean), rstd.data_ptr(), _lib.ptr(dres2),
        dx.data_ptr(), dg.data_ptr(), _lib.ptr(db), scratch.data_ptr(), rows, D, int(rms), int(acc),
        _lib.stream_ptr()), "cgk_norm_backward")
    _lib.count_launch(2)
    return dx, dg, db


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, eps, rms, passthrough=False):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, D)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
        y, s, mean, rstd = norm_forward_raw(x2, gamma, beta, eps, rms, r2, want_sum=True)
        src = s if s is not None else x2
        ctx.save_for_backward(src, gamma, mean, rstd)
        ctx.rms = rms
        ctx.params = (gamma, beta)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        ctx.slot = _lib.grad_slot()
        if residual is not None:
            return y.reshape(x.shape), s.reshape(x.shape)
        if passthrough:
            # the input goes out again as a second result (the residual branch reads it); its gradient
            # comes back as `dsum` and is added inside the backward kernel instead of by autograd
            return y.reshape(x.shape), x.view_as(x)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy, dsum=None):
        src, gamma, mean, rstd = ctx.saved_tensors
        D = src.shape[-1]
        g, b = ctx.params
        dy2 = dy.reshape(-1, D)
        d2 = None
        if dsum is not None:
            d2 = dsum.reshape(-1, D)
            if not d2.is_contiguous():
                d2 = d2.contiguous()
        prev = _lib.set_grad_slot(ctx.slot)
        try:
            mg_g = _lib.main_grad_of(g)
            mg_b = _lib.main_grad_of(b)
            dx, dg, db = norm_backward_raw(dy2, src, gamma, mean, rstd, ctx.rms, d2, mg_g, mg_b)
        finally:
            _lib.set_grad_slot(prev)
        dx = dx.reshape(ctx.shape)
        dgamma = None if mg_g is not None else dg.to(g.dtype)
        dbeta = None
        if b is not None and not ctx.rms:
            dbeta = None if mg_b is not None else db.to(b.dtype)
        return dx, dgamma, dbeta, (dx if ctx.has_res else None), None, None, None


def layer_norm(x, gamma, beta=None, eps: float = 1e-5, residual=None, passthrough: bool = False):
    """``passthrough=True`` (without ``residual``) returns ``(y, x)``: use the second result wherever
    the block reads ``x`` again (its residual branch); the two gradients then meet inside the norm's
    backward kernel instead of in a separate addition."""
    return _Norm.apply(x, gamma, beta, residual, eps, False, passthrough)


def rms_norm(x, gamma, eps: float = 1e-6, residual=None, passthrough: bool = False):
    return _Norm.apply(x, gamma, None, residual, eps, True, passthrough)
