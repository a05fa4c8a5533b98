"""Embedding, SwiGLU, dropout and rotary embedding as differentiable ops.

Reference counterparts: SwiGLU (src/layers/activations.c:17-62: split the last
dimension in halves, ``silu(gate) * value``), inverted dropout (:360-445), RoPE
rotate-half with precomputed ``[max_seq, D/2]`` tables
(src/attention/flash_attn.c:318-362, src/cuda/flash_attn_kernels.c:216-249,656-682).
"""
from __future__ import annotations

import torch

from . import _lib

_BF16 = torch.bfloat16


def _dt(t):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == _BF16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


# ---------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, vocab_start):
        B, T = ids.shape
        D = wte.shape[1]
        ids = ids.contiguous()
        if not wte.is_cuda:
            local = ids - vocab_start
            ok = (local >= 0) & (local < wte.shape[0])
            out = wte[local.clamp(0, wte.shape[0] - 1)] * ok[..., None]
            if wpe is not None:
                out = out + wpe[:T][None]
        else:
            out = torch.empty(B, T, D, device=wte.device, dtype=_BF16)
            _lib.check(_lib.lib().cgk_embedding_forward(
                ids.data_ptr(), wte.data_ptr(), _lib.ptr(wpe), out.data_ptr(), B * T, D, T, int(vocab_start),
                wte.shape[0], _lib.stream_ptr()), "cgk_embedding_forward")
            _lib.count_launch()
        ctx.save_for_backward(ids)
        ctx.params = (wte, wpe)
        ctx.vocab_start = vocab_start
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        wte, wpe = ctx.params
        B, T = ids.shape
        D = wte.shape[1]
        dout = dout.contiguous()
        g_wte = getattr(wte, "main_grad", None)
        g_wpe = getattr(wpe, "main_grad", None) if wpe is not None else None
        own_wte = g_wte is None
        own_wpe = wpe is not None and g_wpe is None
        if own_wte:
            g_wte = torch.zeros(wte.shape, device=wte.device, dtype=torch.float32)
        if own_wpe:
            g_wpe = torch.zeros(wpe.shape, device=wpe.device, dtype=torch.float32)
        if not wte.is_cuda:
            local = (ids - ctx.vocab_start).reshape(-1)
            ok = (local >= 0) & (local < wte.shape[0])
            g_wte.index_add_(0, local[ok], dout.reshape(-1, D).float()[ok])
            if wpe is not None:
                g_wpe[:T] += dout.float().sum(0)
        else:
            _lib.check(_lib.lib().cgk_embedding_backward(
                ids.data_ptr(), dout.data_ptr(), g_wte.data_ptr(), _lib.ptr(g_wpe), B * T, D, T,
                int(ctx.vocab_start), wte.shape[0], _lib.stream_ptr()), "cgk_embedding_backward")
            _lib.count_launch()
        return (None, g_wte.to(wte.dtype) if own_wte else None,
                (g_wpe.to(wpe.dtype) if own_wpe else None), None)


def embedding(ids, wte, wpe=None, vocab_start: int = 0):
    """out[b, t] = wte[ids[b, t] - vocab_start] (+ wpe[t]); ids outside the local
    vocabulary shard contribute zero (vocabulary-parallel embedding)."""
    return _Embedding.apply(ids, wte, wpe, vocab_start)


# ---------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        H = x.shape[-1] // 2
        ctx.save_for_backward(x)
        if not x.is_cuda:
            g, v = x.float()[..., :H], x.float()[..., H:]
            return (torch.nn.functional.silu(g) * v).to(x.dtype)
        x2 = x.reshape(-1, 2 * H).contiguous()
        y = torch.empty(x2.shape[0], H, device=x.device, dtype=x.dtype)
        _lib.check(_lib.lib().cgk_swiglu_forward(_dt(x2), x2.data_ptr(), y.data_ptr(), x2.shape[0], H,
                                                 _lib.stream_ptr()), "cgk_swiglu_forward")
        _lib.count_launch()
        return y.reshape(*x.shape[:-1], H)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        H = x.shape[-1] // 2
        if not x.is_cuda:
            g, v = x.float()[..., :H], x.float()[..., H:]
            s = torch.sigmoid(g)
            dg = dy.float() * v * s * (1 + g * (1 - s))
            dv = dy.float() * g * s
            return torch.cat([dg, dv], -1).to(x.dtype)
        x2 = x.reshape(-1, 2 * H).contiguous()
        dy2 = dy.reshape(-1, H).contiguous()
        dx = torch.empty_like(x2)
        _lib.check(_lib.lib().cgk_swiglu_backward(_dt(x2), x2.data_ptr(), dy2.data_ptr(), dx.data_ptr(),
                                                  x2.shape[0], H, _lib.stream_ptr()), "cgk_swiglu_backward")
        _lib.count_launch()
        return dx.reshape(x.shape)


def swiglu(x):
    """x[..., :H] is the gate, x[..., H:] the value: silu(gate) * value."""
    return _SwiGLU.apply(x)


# ---------------------------------------------------------------------------
class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        return _dropout_apply(x, p, seed)

    @staticmethod
    def backward(ctx, dy):
        return _dropout_apply(dy, ctx.p, ctx.seed), None, None


def _dropout_apply(x, p, seed):
    if not x.is_cuda:
        g = torch.Generator().manual_seed(seed)
        keep = (torch.rand(x.shape, generator=g) >= p).to(x.dtype)
        return x * keep / (1.0 - p)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.lib().cgk_dropout(_dt(x), x.data_ptr(), out.data_ptr(), x.numel(), float(p), int(seed),
                                      _lib.stream_ptr()), "cgk_dropout")
    _lib.count_launch()
    return out


_dropout_counter = [0]


def dropout(x, p: float, training: bool = True, seed: int | None = None):
    """Inverted dropout; the mask is a function of (seed, element index) so the
    backward pass regenerates it instead of storing it."""
    if not training or p <= 0.0:
        return x
    if seed is None:
        _dropout_counter[0] += 1
        seed = (torch.initial_seed() * 1000003 + _dropout_counter[0]) & 0x7FFFFFFFFFFFFFFF
    return _Dropout.apply(x, p, seed)


class _SoftmaxDropoutResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mul, residual, p, seed):
        V = x.shape[-1]
        x2 = x.reshape(-1, V).contiguous()
        ctx.p, ctx.seed, ctx.has_res = p, seed, residual is not None
        m2 = mul.reshape(-1, V).contiguous() if mul is not None else None
        ctx.save_for_backward(x2, m2 if m2 is not None else torch.empty(0))
        ctx.has_mul = mul is not None
        ctx.shape = x.shape
        if not x.is_cuda:
            s = torch.softmax(x2.float(), -1)
            w = mul.reshape(-1, V).float() if mul is not None else _keep_cpu(x2.shape, p, seed)
            out = s * w
            if residual is not None:
                out = out + residual.reshape(-1, V).float()
            return out.to(x.dtype).reshape(x.shape)
        out = torch.empty_like(x2)
        r2 = residual.reshape(-1, V).contiguous() if residual is not None else None
        _lib.check(_lib.lib().cgk_softmax_dropout_residual(_dt(x2), x2.data_ptr(), _lib.ptr(m2), _lib.ptr(r2), out.data_ptr(),
                                                           x2.shape[0], V, float(p), int(seed), _lib.stream_ptr()),
                   "cgk_softmax_dropout_residual")
        _lib.count_launch()
        return out.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, m2 = ctx.saved_tensors
        V = x2.shape[-1]
        dy2 = dy.reshape(-1, V).contiguous()
        mul = m2 if ctx.has_mul else None
        if not x2.is_cuda:
            s = torch.softmax(x2.float(), -1)
            w = mul.float() if mul is not None else _keep_cpu(x2.shape, ctx.p, ctx.seed)
            g = dy2.float() * w
            dx = (s * (g - (g * s).sum(-1, keepdim=True))).to(x2.dtype)
        else:
            dx = torch.empty_like(x2)
            _lib.check(_lib.lib().cgk_softmax_dropout_residual_backward(_dt(x2), x2.data_ptr(), _lib.ptr(mul), dy2.data_ptr(),
                                                                        dx.data_ptr(), x2.shape[0], V, float(ctx.p), int(ctx.seed),
                                                                        _lib.stream_ptr()), "cgk_softmax_dropout_residual_backward")
            _lib.count_launch()
        return dx.reshape(ctx.shape), None, (dy if ctx.has_res else None), None, None


def _keep_cpu(shape, p, seed):
    if p <= 0.0:
        return torch.ones(shape)
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(shape, generator=g) >= p).float() / (1.0 - p)


def softmax_dropout_residual(x, residual=None, p: float = 0.0, training: bool = True, seed: int | None = None, mul=None):
    """``dropout(softmax(x, -1), p) + residual`` as one pass over each row (fp32 or bf16).  With ``mul``
    the softmax is multiplied by that tensor instead of a generated mask: the softmax -> mul -> add
    chain that the fusion pass names ``fused_softmax_dropout_residual`` (src/jit/fusion.c:152-190 in
    the reference, where it is a name only).  The backward pass recomputes the softmax from ``x`` and
    regenerates the mask from the seed; ``mul`` itself gets no gradient."""
    if not training:
        p = 0.0
    if seed is None:
        _dropout_counter[0] += 1
        seed = (torch.initial_seed() * 1000003 + _dropout_counter[0]) & 0x7FFFFFFFFFFFFFFF
    return _SoftmaxDropoutResidual.apply(x, mul, residual, float(p), seed)


# ---------------------------------------------------------------------------
def rope_tables(max_seq: int, head_dim: int, theta: float = 10000.0, device=None):
    """cos / sin tables [max_seq, head_dim / 2], angle = pos * theta^(-2i/D)."""
    half = head_dim // 2
    dev = torch.device(device) if device is not None else torch.device("cpu")
    if dev.type != "cuda":
        inv = theta ** (-torch.arange(half, dtype=torch.float32) * 2.0 / head_dim)
        ang = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv[None]
        return torch.cos(ang).to(dev), torch.sin(ang).to(dev)
    cos_t = torch.empty(max_seq, half, device=dev, dtype=torch.float32)
    sin_t = torch.empty(max_seq, half, device=dev, dtype=torch.float32)
    _lib.check(_lib.lib().cgk_rope_table(cos_t.data_ptr(), sin_t.data_ptr(), max_seq, head_dim, float(theta),
                                         _lib.stream_ptr()), "cgk_rope_table")
    _lib.count_launch()
    return cos_t, sin_t


def rope_apply_(x, cos_t, sin_t, pos_offset: int = 0, positions=None, backward: bool = False):
    """In-place rotation of x [B, T, H, D] (strided views allowed, D contiguous)."""
    B, T, H, D = x.shape
    half = D // 2
    if not x.is_cuda:
        pos = positions.long() if positions is not None else (torch.arange(T) + pos_offset)[None].expand(B, T)
        pos = pos.clamp(0, cos_t.shape[0] - 1)
        c = cos_t[pos][:, :, None, :]
        s = sin_t[pos][:, :, None, :] * (-1.0 if backward else 1.0)
        a, b = x[..., :half].float().clone(), x[..., half:].float().clone()
        x[..., :half] = (a * c - b * s).to(x.dtype)
        x[..., half:] = (b * c + a * s).to(x.dtype)
        return x
    assert x.stride(3) == 1
    L = _lib.lib()
    if positions is not None:
        positions = positions.to(torch.int32).contiguous()
    _lib.check(L.cgk_rope_apply(_dt(x), x.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), _lib.ptr(positions),
                                B, T, H, D, x.stride(0), x.stride(1), x.stride(2), int(pos_offset),
                                cos_t.shape[0], int(backward), _lib.stream_ptr()), "cgk_rope_apply")
    _lib.count_launch()
    return x


class _RopeQK(torch.autograd.Function):
    """Rotate the q and k slices of a packed projection in place."""

    @staticmethod
    def forward(ctx, x, cos_t, sin_t, nrot, pos_offset):
        # x: [B, T, Htot, D]; the first nrot heads are rotated (q heads then k heads)
        ctx.save_for_backward(cos_t, sin_t)
        ctx.nrot, ctx.pos_offset = nrot, pos_offset
        ctx.mark_dirty(x)
        rope_apply_(x[:, :, :nrot], cos_t, sin_t, pos_offset)
        return x

    @staticmethod
    def backward(ctx, dx):
        cos_t, sin_t = ctx.saved_tensors
        dx = dx.contiguous() if not dx.is_contiguous() else dx.clone()
        rope_apply_(dx[:, :, :ctx.nrot], cos_t, sin_t, ctx.pos_offset, backward=True)
        return dx, None, None, None, None


def rope_qk_(x, cos_t, sin_t, nrot: int, pos_offset: int = 0):
    """x: [B, T, heads_total, D] holding q heads, k heads, v heads in that order;
    rotates the first `nrot` heads in place (differentiable)."""
    return _RopeQK.apply(x, cos_t, sin_t, nrot, pos_offset)
