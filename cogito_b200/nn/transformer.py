"""Attention and transformer block.

The block follows cg_transformer_config (include/cg_transformer.h:19-34: hidden,
heads, kv_heads, head_dim, intermediate, eps, dropout, bias, pre_norm, rms_norm,
swiglu) and the forward order of transformer_forward
(src/layers/transformer.c:26-149): norm -> q,k,v projection -> flash attention ->
output projection -> dropout -> residual -> norm -> MLP (SwiGLU gate/up/down, or
up/activation/down) -> dropout -> residual.  The reference calls an undefined
attention function and has no backward; this one trains.

Fusions on the CUDA path: one QKV GEMM; RoPE applied in place on the packed
projection; attention reads q/k/v as strided views of that buffer and its backward
writes dq/dk/dv into one packed gradient; residual adds ride in the epilogue of the
output-projection and MLP-down GEMMs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from ..ops import functional as F
from ..ops import misc as M
from ..ops.attention import alibi_slopes, flash_backward, flash_forward
from ..ops.gemm import gemm
from .modules import Dropout, LayerNorm, Linear, RMSNorm, _maybe_bf16


@dataclass
class TransformerConfig:
    hidden_size: int = 768
    num_heads: int = 12
    num_kv_heads: int | None = None      # None: same as num_heads (MHA)
    head_dim: int | None = None          # None: hidden_size // num_heads
    intermediate_size: int = 3072
    norm_eps: float = 1e-5
    dropout: float = 0.0
    bias: bool = True
    pre_norm: bool = True
    rms_norm: bool = False
    swiglu: bool = False
    activation: str = "gelu"             # used when swiglu is False
    causal: bool = True
    window: int = -1
    rope: bool = False
    rope_theta: float = 10000.0
    alibi: bool = False
    max_seq_len: int = 2048
    init_std: float = 0.02

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_heads


class _PackedAttention(torch.autograd.Function):
    """x: [B, T, Hq + 2*Hk, D] = q heads | k heads | v heads."""

    @staticmethod
    def forward(ctx, x, Hq, Hk, causal, window, scale, alibi, rope):
        # RoPE rotates the q and k heads of the projection buffer in place; the
        # producer (a GEMM) does not need its own output for its backward, so
        # autograd is not told.  The rotated buffer is what gets saved.
        if rope is not None:
            M.rope_apply_(x.data[:, :, :Hq + Hk], rope[0], rope[1])   # .data: no version bump
        q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hk], x[:, :, Hq + Hk:]
        o, lse = flash_forward(q, k, v, causal=causal, window=window, scale=scale, alibi=alibi)
        ctx.save_for_backward(x, o, lse, alibi if alibi is not None else torch.empty(0))
        ctx.cfg = (Hq, Hk, causal, window, scale, alibi is not None)
        ctx.rope = rope
        return o

    @staticmethod
    def backward(ctx, do):
        x, o, lse, alibi = ctx.saved_tensors
        Hq, Hk, causal, window, scale, has_alibi = ctx.cfg
        q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hk], x[:, :, Hq + Hk:]
        dx = torch.empty_like(x)
        kw = dict(causal=causal, window=window, scale=scale, alibi=alibi if has_alibi else None)
        if x.is_cuda:
            flash_backward(do, q, k, v, o, lse, dq=dx[:, :, :Hq], dk=dx[:, :, Hq:Hq + Hk],
                           dv=dx[:, :, Hq + Hk:], **kw)
        else:
            dq, dk, dv = flash_backward(do, q, k, v, o, lse, **kw)
            dx[:, :, :Hq], dx[:, :, Hq:Hq + Hk], dx[:, :, Hq + Hk:] = dq, dk, dv
        if ctx.rope is not None:
            M.rope_apply_(dx[:, :, :Hq + Hk], ctx.rope[0], ctx.rope[1], backward=True)
        return dx, None, None, None, None, None, None, None


class _QKVRopeAttention(torch.autograd.Function):
    """o = attention(rope(h W^T + b)): the QKV projection applies the rotary embedding to its q and
    k columns in the GEMM's epilogue (no separate pass over the projection), attention runs on the
    packed result, and the backward pass undoes the rotation on the gradient of the projection (in
    place, on its own buffer) before the two backward GEMMs.
    Reference: OP_FUSED_QKV_ROPE (include/cg_jit.h:59, src/jit/fusion.c:192-224, a name only there)
    and cg_flash_attention_forward_rope_cuda (src/cuda/flash_attn_kernels.c:568)."""

    @staticmethod
    def forward(ctx, h, w, b, Hq, Hk, D, causal, window, scale, alibi, rope):
        B, T, _ = h.shape
        x2 = h.reshape(B * T, -1)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        spec = (rope[0], rope[1], (Hq + Hk) * D, D, T, 0, False)
        qkv = gemm(x2, w, bias=b, rope=spec).view(B, T, Hq + 2 * Hk, D)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:]
        o, lse = flash_forward(q, k, v, causal=causal, window=window, scale=scale, alibi=alibi)
        ctx.save_for_backward(x2, w, qkv, o, lse, alibi if alibi is not None else torch.empty(0))
        ctx.cfg = (Hq, Hk, D, causal, window, scale, alibi is not None)
        ctx.rope, ctx.bias, ctx.hshape = rope, b, h.shape
        return o

    @staticmethod
    def backward(ctx, do):
        x2, w, qkv, o, lse, alibi = ctx.saved_tensors
        Hq, Hk, D, causal, window, scale, has_alibi = ctx.cfg
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:]
        dqkv = torch.empty_like(qkv)
        kw = dict(causal=causal, window=window, scale=scale, alibi=alibi if has_alibi else None)
        if qkv.is_cuda:
            flash_backward(do.contiguous(), q, k, v, o, lse, dq=dqkv[:, :, :Hq], dk=dqkv[:, :, Hq:Hq + Hk],
                           dv=dqkv[:, :, Hq + Hk:], **kw)
        else:
            dq, dk, dv = flash_backward(do, q, k, v, o, lse, **kw)
            dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hk], dqkv[:, :, Hq + Hk:] = dq, dk, dv
        M.rope_apply_(dqkv[:, :, :Hq + Hk], ctx.rope[0], ctx.rope[1], backward=True)
        d2 = dqkv.view(x2.shape[0], -1)
        dh = gemm(d2, w, b_mn=True).view(ctx.hshape) if ctx.needs_input_grad[0] else None
        dw = F._weight_grad(d2, x2, w)
        db = F._bias_grad(d2, ctx.bias) if ctx.bias is not None else None
        return dh, dw, db, None, None, None, None, None, None, None, None


def packed_attention(x, Hq, Hk, *, causal=True, window=-1, scale=None, alibi=None, rope=None):
    """rope: (cos, sin) tables or None; positions are 0..T-1."""
    return _PackedAttention.apply(x, Hq, Hk, causal, window, scale, alibi, rope)


class SelfAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        Hq, Hk, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        self.qkv = Linear(cfg.hidden_size, (Hq + 2 * Hk) * D, bias=cfg.bias, init_std=cfg.init_std,
                          device=device, dtype=dtype)
        self.proj = Linear(Hq * D, cfg.hidden_size, bias=cfg.bias, init_std=cfg.init_std,
                           device=device, dtype=dtype)
        self._rope = None
        self._alibi = None

    def _tables(self, device):
        if self.cfg.rope and (self._rope is None or self._rope[0].device != device):
            self._rope = M.rope_tables(self.cfg.max_seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        if self.cfg.alibi and (self._alibi is None or self._alibi.device != device):
            self._alibi = alibi_slopes(self.cfg.num_heads, device)

    def forward(self, h, residual=None):
        cfg = self.cfg
        B, T, _ = h.shape
        Hq, Hk, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        self._tables(h.device)
        if cfg.rope and h.is_cuda and D in (64, 128) and h.dtype == torch.bfloat16:
            o = _QKVRopeAttention.apply(h, self.qkv.weight, self.qkv.bias, Hq, Hk, D, cfg.causal, cfg.window,
                                        1.0 / math.sqrt(D), self._alibi, self._rope)
            return self.proj(o.reshape(B, T, Hq * D), residual=residual)
        x = self.qkv(h).view(B, T, Hq + 2 * Hk, D)
        o = packed_attention(x, Hq, Hk, causal=cfg.causal, window=cfg.window,
                             scale=1.0 / math.sqrt(D), alibi=self._alibi,
                             rope=self._rope if cfg.rope else None)
        return self.proj(o.reshape(B, T, Hq * D), residual=residual)


class FeedForward(nn.Module):
    def __init__(self, cfg: TransformerConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        if cfg.swiglu:
            self.gate_up = Linear(cfg.hidden_size, 2 * cfg.intermediate_size, bias=cfg.bias,
                                  init_std=cfg.init_std, device=device, dtype=dtype)
        else:
            self.up = Linear(cfg.hidden_size, cfg.intermediate_size, bias=cfg.bias, init_std=cfg.init_std,
                             device=device, dtype=dtype)
        self.down = Linear(cfg.intermediate_size, cfg.hidden_size, bias=cfg.bias, init_std=cfg.init_std,
                           device=device, dtype=dtype)

    def forward(self, h, residual=None):
        if self.cfg.swiglu:
            return self.down(M.swiglu(self.gate_up(h)), residual=residual)
        h = _maybe_bf16(h)
        return F.mlp(h, self.up.weight, self.up.bias, self.down.weight, self.down.bias,
                     self.cfg.activation, residual)


class TransformerBlock(nn.Module):
    def __init__(self, cfg: TransformerConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        Norm = (lambda: RMSNorm(cfg.hidden_size, cfg.norm_eps, device=device, dtype=dtype)) if cfg.rms_norm \
            else (lambda: LayerNorm(cfg.hidden_size, cfg.norm_eps, device=device, dtype=dtype))
        self.norm1 = Norm()
        self.attn = SelfAttention(cfg, device, dtype)
        self.norm2 = Norm()
        self.mlp = FeedForward(cfg, device, dtype)
        self.drop = Dropout(cfg.dropout)

    def forward(self, x):
        cfg = self.cfg
        if cfg.pre_norm:
            if cfg.dropout > 0 and self.training:
                x = x + self.drop(self.attn(self.norm1(x)))
                return x + self.drop(self.mlp(self.norm2(x)))
            # the norm hands its input back as a second result for the residual branch, so that the
            # two gradients of x are summed inside the norm's backward kernel
            h, xr = self.norm1(x, passthrough=True)
            x = self.attn(h, residual=xr)
            h, xr = self.norm2(x, passthrough=True)
            return self.mlp(h, residual=xr)
        # post-norm: x = norm(x + f(x))
        x = self.norm1(x + self.drop(self.attn(x)))
        return self.norm2(x + self.drop(self.mlp(x)))
