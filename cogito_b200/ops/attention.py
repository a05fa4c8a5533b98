"""Flash-Attention-2 forward / backward (tcgen05 kernels) and its fp32 oracle.

Tensors use the reference's layout ``[batch, seq, heads, head_dim]``
(include/cg_flash_attn.h:54-57); LSE is ``[batch, heads, seq]`` (:81).
The functions the reference declares but never defines —
``cg_flash_attention_forward/backward/mqa/gqa`` (include/cg_flash_attn.h) — map
onto :func:`flash_attention` with the matching head counts.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import POINTER, Structure, c_float, c_int32, c_int64, c_void_p

import torch

from . import _lib


class FlashArgs(Structure):
    """Mirror of ``cgk_flash_args`` (include/cogito_kernels.h)."""

    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
        ("B", c_int32), ("Hq", c_int32), ("Hk", c_int32), ("Tq", c_int32), ("Tk", c_int32), ("D", c_int32),
        ("q_bs", c_int64), ("q_ts", c_int64), ("q_hs", c_int64),
        ("k_bs", c_int64), ("k_ts", c_int64), ("k_hs", c_int64),
        ("v_bs", c_int64), ("v_ts", c_int64), ("v_hs", c_int64),
        ("o_bs", c_int64), ("o_ts", c_int64), ("o_hs", c_int64),
        ("scale", c_float), ("causal", c_int32), ("window", c_int32),
        ("alibi_slopes", c_void_p),
        ("d_o", c_void_p), ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("dq_bs", c_int64), ("dq_ts", c_int64), ("dq_hs", c_int64),
        ("dk_bs", c_int64), ("dk_ts", c_int64), ("dk_hs", c_int64),
        ("dv_bs", c_int64), ("dv_ts", c_int64), ("dv_hs", c_int64),
        ("delta", c_void_p), ("dq_accum", c_void_p),
    ]


_declared = False


def _fns():
    global _declared
    L = _lib.lib()
    if not _declared:
        L.cgk_flash_forward.argtypes = [POINTER(FlashArgs), c_void_p]
        L.cgk_flash_backward.argtypes = [POINTER(FlashArgs), c_void_p]
        _declared = True
    return L


def alibi_slopes(num_heads: int, device=None) -> torch.Tensor:
    """Slopes 2^(-8 (h+1) / H), as cg_alibi_slopes (src/attention/flash_attn.c:368-388)."""
    h = torch.arange(1, num_heads + 1, dtype=torch.float32, device=device)
    return torch.pow(2.0, -8.0 * h / num_heads)


def attention_reference(q, k, v, *, causal=False, window=-1, scale=None, alibi=None):
    """Naive softmax(QK^T)V in fp32 with the same masking rules; returns (o, lse)."""
    B, Tq, Hq, D = q.shape
    Tk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hk
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    qi = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
    ki = torch.arange(Tk, device=q.device)[None, :]
    if alibi is not None:
        s = s + alibi.float().view(1, Hq, 1, 1) * (ki - qi).float()
    vis = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        vis &= ki <= qi
    if window is not None and window >= 0:
        vis &= (ki - qi).abs() <= window
    s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(torch.isinf(lse), 0.0).unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    lse = torch.where(torch.isinf(lse), torch.full_like(lse, float("inf")), lse)
    return o, lse


def _strides3(t):
    assert t.stride(3) == 1, "head_dim must be contiguous"
    return t.stride(0), t.stride(1), t.stride(2)


def _fill_common(a: FlashArgs, q, k, v, o, lse, scale, causal, window, alibi):
    B, Tq, Hq, D = q.shape
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr()
    a.B, a.Hq, a.Hk, a.Tq, a.Tk, a.D = B, Hq, k.shape[2], Tq, k.shape[1], D
    a.q_bs, a.q_ts, a.q_hs = _strides3(q)
    a.k_bs, a.k_ts, a.k_hs = _strides3(k)
    a.v_bs, a.v_ts, a.v_hs = _strides3(v)
    a.o_bs, a.o_ts, a.o_hs = _strides3(o)
    a.scale = float(scale)
    a.causal = int(bool(causal))
    a.window = int(window if window is not None else -1)
    a.alibi_slopes = alibi.data_ptr() if alibi is not None else None


def flash_forward(q, k, v, *, causal=False, window=-1, scale=None, alibi=None):
    """Returns (o [B,Tq,Hq,D] bf16, lse [B,Hq,Tq] fp32).  q/k/v may be strided views."""
    B, Tq, Hq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        o, lse = attention_reference(q, k, v, causal=causal, window=window, scale=scale, alibi=alibi)
        return o.to(q.dtype), lse
    if q.dtype != torch.bfloat16:
        raise TypeError("flash_forward: CUDA tensors must be bf16")
    o = torch.empty(B, Tq, Hq, D, device=q.device, dtype=torch.bfloat16)
    lse = torch.empty(B, Hq, Tq, device=q.device, dtype=torch.float32)
    a = FlashArgs()
    _fill_common(a, q, k, v, o, lse, scale, causal, window, alibi)
    _lib.check(_fns().cgk_flash_forward(ctypes.byref(a), _lib.stream_ptr()), "cgk_flash_forward")
    _lib.count_launch()
    return o, lse


def flash_backward(do, q, k, v, o, lse, *, causal=False, window=-1, scale=None, alibi=None,
                   dq=None, dk=None, dv=None):
    """Gradients of :func:`flash_forward`.  dq/dk/dv may be preallocated strided views."""
    B, Tq, Hq, D = q.shape
    Tk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            oo, _ = attention_reference(qq, kk, vv, causal=causal, window=window, scale=scale, alibi=alibi)
            gq, gk, gv = torch.autograd.grad(oo, (qq, kk, vv), do.float())
        return gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype)
    if do.stride() != o.stride():
        do = do.contiguous()
        if do.stride() != o.stride():
            o = o.contiguous()
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    delta = torch.empty(B, Hq, Tq, device=q.device, dtype=torch.float32)
    dq_accum = torch.empty(B, Tq, Hq, D, device=q.device, dtype=torch.float32)
    a = FlashArgs()
    _fill_common(a, q, k, v, o, lse, scale, causal, window, alibi)
    a.d_o = do.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_bs, a.dq_ts, a.dq_hs = _strides3(dq)
    a.dk_bs, a.dk_ts, a.dk_hs = _strides3(dk)
    a.dv_bs, a.dv_ts, a.dv_hs = _strides3(dv)
    a.delta, a.dq_accum = delta.data_ptr(), dq_accum.data_ptr()
    _lib.check(_fns().cgk_flash_backward(ctypes.byref(a), _lib.stream_ptr()), "cgk_flash_backward")
    _lib.count_launch(4)
    return dq, dk, dv


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, alibi):
        o, lse = flash_forward(q, k, v, causal=causal, window=window, scale=scale, alibi=alibi)
        ctx.save_for_backward(q, k, v, o, lse, alibi if alibi is not None else torch.empty(0))
        ctx.cfg = (causal, window, scale, alibi is not None)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, alibi = ctx.saved_tensors
        causal, window, scale, has_alibi = ctx.cfg
        dq, dk, dv = flash_backward(do, q, k, v, o, lse, causal=causal, window=window, scale=scale,
                                    alibi=alibi if has_alibi else None)
        return dq, dk, dv, None, None, None, None


def flash_attention(q, k, v, *, causal=False, window=-1, scale=None, alibi=None):
    """Differentiable attention.  q: [B,Tq,Hq,D]; k, v: [B,Tk,Hk,D] with Hq % Hk == 0
    (Hk == Hq: MHA, Hk == 1: MQA, otherwise GQA)."""
    return _FlashAttn.apply(q, k, v, causal, window, scale, alibi)


class _FlashAttnPacked(torch.autograd.Function):
    """Attention over a packed ``qkv`` tensor [B, T, 3, H, D]; the backward writes the
    three gradients straight into one [B, T, 3, H, D] buffer (no concatenation)."""

    @staticmethod
    def forward(ctx, qkv, causal, window, scale, alibi):
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        o, lse = flash_forward(q, k, v, causal=causal, window=window, scale=scale, alibi=alibi)
        ctx.save_for_backward(qkv, o, lse, alibi if alibi is not None else torch.empty(0))
        ctx.cfg = (causal, window, scale, alibi is not None)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, alibi = ctx.saved_tensors
        causal, window, scale, has_alibi = ctx.cfg
        dqkv = torch.empty_like(qkv)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if qkv.is_cuda:
            flash_backward(do, q, k, v, o, lse, causal=causal, window=window, scale=scale,
                           alibi=alibi if has_alibi else None,
                           dq=dqkv[:, :, 0], dk=dqkv[:, :, 1], dv=dqkv[:, :, 2])
        else:
            dq, dk, dv = flash_backward(do, q, k, v, o, lse, causal=causal, window=window, scale=scale,
                                        alibi=alibi if has_alibi else None)
            dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2] = dq, dk, dv
        return dqkv, None, None, None, None


def flash_attention_qkvpacked(qkv, *, causal=False, window=-1, scale=None, alibi=None):
    """qkv: [B, T, 3, H, D] (as produced by a fused QKV projection). Returns [B, T, H, D]."""
    return _FlashAttnPacked.apply(qkv, causal, window, scale, alibi)
