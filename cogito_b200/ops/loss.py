"""Losses.  The large-vocabulary path is a fused softmax-cross-entropy kernel that
produces the loss and d(logits) in one launch (d(logits) overwrites the logits).

The small losses keep the reference's definitions (src/layers/loss.c): MSE
(:14-39), cross-entropy over softmax with a 1e-7 clamp (:44-78), BCE (:87-113),
L1 (:118-142), BCE-with-logits in its stable form (:147-175) and the
``cg_smooth_l1_loss`` the reference declares (include/cg_loss.h:119-120) but
never defines.  Reductions: "mean", "sum" ("none" gives per-element values).
"""
from __future__ import annotations

import torch

from . import _lib

_BF16 = torch.bfloat16


class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, grad_scale, ignore_index):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        t1 = targets.reshape(-1)
        R = l2.shape[0]
        valid = (t1 != ignore_index)
        if not logits.is_cuda:
            lf = l2.float()
            lse = torch.logsumexp(lf, -1)
            tgt = t1.clamp(min=0)
            rows = (lse - lf.gather(1, tgt[:, None]).squeeze(1)) * valid
            n = valid.sum().clamp(min=1)
            p = torch.softmax(lf, -1)
            p[torch.arange(R), tgt] -= 1.0
            d = p * valid[:, None] * (float(grad_scale) / n)
            ctx.save_for_backward(d.to(logits.dtype))
            ctx.shape = logits.shape
            return rows.sum() / n
        if l2.dtype != _BF16 or l2.stride(-1) != 1:
            raise TypeError("cross_entropy: CUDA logits must be bf16 with a contiguous last dimension")
        n_valid = valid.sum().clamp(min=1).float()
        inv_n = (1.0 / n_valid).reshape(1)
        rows = torch.empty(R, device=logits.device, dtype=torch.float32)
        t1 = t1.contiguous()
        if isinstance(grad_scale, torch.Tensor):
            inv_n = inv_n * grad_scale.reshape(1).float()   # device-resident loss scale: no host sync
            scale_f = 1.0
        else:
            scale_f = float(grad_scale)
        _lib.check(_lib.lib().cgk_softmax_ce_fused(
            l2.data_ptr(), t1.data_ptr(), rows.data_ptr(), l2.data_ptr(), R, V, l2.stride(0), scale_f,
            _lib.ptr(inv_n), int(ignore_index), _lib.stream_ptr()), "cgk_softmax_ce_fused")
        _lib.count_launch()
        ctx.save_for_backward(l2)      # now holds d(logits)
        ctx.shape = logits.shape
        return rows.sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d.reshape(ctx.shape), None, None, None


def cross_entropy(logits, targets, grad_scale=1.0, ignore_index: int = -100):
    """Mean cross-entropy of ``logits [..., V]`` against integer ``targets [...]``.

    CUDA: one fused kernel; the logits tensor is overwritten with its own gradient
    ``(softmax - onehot) * grad_scale / n`` and the backward returns it as is, so the
    incoming gradient is taken to be 1 — put a loss scale into ``grad_scale`` (a float,
    or a one-element device tensor such as ``GradScaler.scale_tensor``).
    """
    return _FusedCE.apply(logits, targets, grad_scale, ignore_index)


def _reduce(x, reduction):
    if reduction == "mean":
        return x.mean()
    if reduction == "sum":
        return x.sum()
    return x


def mse_loss(pred, target, reduction="mean"):
    return _reduce((pred - target) ** 2, reduction)


def l1_loss(pred, target, reduction="mean"):
    return _reduce((pred - target).abs(), reduction)


def smooth_l1_loss(pred, target, beta: float = 1.0, reduction="mean"):
    d = (pred - target).abs()
    return _reduce(torch.where(d < beta, 0.5 * d * d / beta, d - 0.5 * beta), reduction)


def bce_loss(prob, target, reduction="mean", eps: float = 1e-7):
    p = prob.clamp(eps, 1.0 - eps)
    return _reduce(-(target * torch.log(p) + (1.0 - target) * torch.log(1.0 - p)), reduction)


def bce_with_logits_loss(logits, target, reduction="mean"):
    # max(x, 0) - x*t + log(1 + exp(-|x|))
    return _reduce(logits.clamp(min=0) - logits * target + torch.log1p(torch.exp(-logits.abs())), reduction)


def softmax_cross_entropy_small(logits, target, reduction="mean", eps: float = 1e-7):
    """The reference's CE for small class counts: target is either class indices or
    a one-hot / probability matrix; probabilities are clamped at 1e-7 before the log.
    The reduction divides by the batch size (rows), not by the element count."""
    p = torch.softmax(logits.float(), -1).clamp(min=eps)
    if target.dtype in (torch.int64, torch.int32):
        rows = -torch.log(p.gather(-1, target.long().unsqueeze(-1)).squeeze(-1))
    else:
        rows = -(target.float() * torch.log(p)).sum(-1)
    return _reduce(rows, reduction)
