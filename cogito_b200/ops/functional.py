"""Differentiable ops built on the sm_100a kernels (CUDA) with an fp32 PyTorch
restatement for CPU tensors.  These are what the ``nn`` modules call.

Weight gradients: when a parameter carries a ``main_grad`` attribute (an fp32
view into the optimizer's flat gradient buffer) the backward GEMM accumulates
straight into it from the epilogue and autograd receives ``None`` for that
parameter; otherwise an ordinary gradient tensor is returned.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .gemm import gemm

_BF16 = torch.bfloat16


def _use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda


def _scratch(n: int, device, dtype=torch.float32) -> torch.Tensor:
    return torch.empty(max(int(n), 1), device=device, dtype=dtype)


# ---------------------------------------------------------------------------
# helpers shared by the linear-type backward passes
# ---------------------------------------------------------------------------
def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
    """dW[N, K] = dy2[M, N]^T @ x2[M, K].  Returns None when accumulated into main_grad."""
    mg = _lib.main_grad_of(w)
    if mg is not None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype if w.dtype == _BF16 else torch.float32)


def colsum(dy2: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Column sums of a bf16 [M, N] matrix into fp32 [N]."""
    M, N = dy2.shape
    if out is None:
        out = torch.empty(N, device=dy2.device, dtype=torch.float32)
        accumulate = False
    if not dy2.is_cuda:
        s = dy2.float().sum(0)
        out.copy_(out + s if accumulate else s)
        return out
    L = _lib.lib()
    if dy2.stride(1) != 1:
        dy2 = dy2.contiguous()
    scratch = _scratch(L.cgk_colsum_scratch_elems(M, N), dy2.device)
    _lib.check(L.cgk_colsum_bf16(dy2.data_ptr(), M, N, dy2.stride(0), out.data_ptr(), scratch.data_ptr(),
                                 int(accumulate), _lib.stream_ptr()), "cgk_colsum_bf16")
    _lib.count_launch(2)
    return out


def _bias_grad(dy2: torch.Tensor, b: torch.Tensor | None):
    if b is None:
        return None
    mg = _lib.main_grad_of(b)
    if mg is not None:
        colsum(dy2, out=mg, accumulate=True)
        return None
    return colsum(dy2).to(b.dtype)


class _Linear(torch.autograd.Function):
    """y = act(x @ W^T + b) (+ residual);  W is [out, in] like torch.nn.Linear."""

    @staticmethod
    def forward(ctx, x, w, b, act, residual):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        need_aux = act not in (None, "none") and (x.requires_grad or w.requires_grad)
        aux = torch.empty(x2.shape[0], w.shape[0], device=x.device, dtype=x.dtype) if need_aux else None
        y = gemm(x2, w, bias=b, act=act, residual=r2, aux_out=aux)
        ctx.save_for_backward(x2, w, aux if aux is not None else torch.empty(0))
        ctx.act = act
        ctx.has_bias = b is not None
        ctx.bias = b
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, aux = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        if ctx.act not in (None, "none"):
            dy2 = unary_backward(ctx.act, aux, dy2)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.xshape)
        dw = _weight_grad(dy2, x2, w) if ctx.needs_input_grad[1] else None
        db = _bias_grad(dy2, ctx.bias) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, dres


def linear(x, w, b=None, act=None, residual=None):
    if x.dtype != _BF16 and x.is_cuda:
        raise TypeError("linear: CUDA activations must be bf16 (use autocast() or .bfloat16())")
    return _Linear.apply(x, w, b, act, residual)


class _MLP(torch.autograd.Function):
    """out = residual + act(x W1^T + b1) W2^T + b2 with a hand-scheduled backward:
    the dX GEMM of the second layer multiplies by act'(z) in its epilogue, so the
    activation gradient never makes a separate pass over memory."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act, residual):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M = x2.shape[0]
        z = torch.empty(M, w1.shape[0], device=x.device, dtype=x.dtype)
        h = gemm(x2, w1, bias=b1, act=act, aux_out=z)
        r2 = residual.reshape(M, -1) if residual is not None else None
        y = gemm(h, w2, bias=b2, residual=r2)
        ctx.save_for_backward(x2, w1, w2, z, h)
        ctx.act = act
        ctx.b1, ctx.b2 = b1, b2
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, z, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, w2.shape[0])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        dw2 = _weight_grad(dy2, h, w2)
        db2 = _bias_grad(dy2, ctx.b2)
        dz = gemm(dy2, w2, b_mn=True, aux_in=z, dact=ctx.act)       # (dy W2) * act'(z)
        dw1 = _weight_grad(dz, x2, w1)
        db1 = _bias_grad(dz, ctx.b1)
        dx = gemm(dz, w1, b_mn=True).reshape(ctx.xshape) if ctx.needs_input_grad[0] else None
        return dx, dw1, db1, dw2, db2, None, dres


def mlp(x, w1, b1, w2, b2, act="gelu", residual=None):
    return _MLP.apply(x, w1, b1, w2, b2, act, residual)


# ---------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------
UNARY = {"exp": 0, "log": 1, "sqrt": 2, "abs": 3, "neg": 4, "rsqrt": 5, "relu": 6, "sigmoid": 7,
         "tanh": 8, "gelu": 9, "silu": 10, "pow": 11, "scale": 12, "adds": 13, "copy": 14,
         "square": 15, "recip": 16}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == _BF16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


def _unary_cpu(op, x, s):
    f = {"exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "abs": torch.abs, "neg": torch.neg,
         "rsqrt": torch.rsqrt, "relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
         "gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
         "silu": torch.nn.functional.silu, "pow": lambda t: torch.pow(t, s),
         "scale": lambda t: t * s, "adds": lambda t: t + s, "copy": lambda t: t.clone(),
         "square": lambda t: t * t, "recip": lambda t: 1.0 / t}[op]
    return f(x.float()).to(x.dtype)


def unary(op: str, x: torch.Tensor, s: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Elementwise f(x); `s` is the exponent / factor / addend of pow, scale, adds."""
    if not x.is_cuda:
        r = _unary_cpu(op, x, s)
        if out is not None:
            out.copy_(r)
            return out
        return r
    x = x.contiguous()
    out = torch.empty_like(x) if out is None else out
    _lib.check(_lib.lib().cgk_unary(UNARY[op], _dt(x), x.data_ptr(), out.data_ptr(), x.numel(), float(s),
                                    _lib.stream_ptr()), "cgk_unary")
    _lib.count_launch()
    return out


def unary_backward(op: str, x: torch.Tensor, dy: torch.Tensor, s: float = 0.0) -> torch.Tensor:
    """dy * f'(x), with x the forward input."""
    if not x.is_cuda:
        xx = x.detach().float().requires_grad_(True)
        with torch.enable_grad():
            y = _unary_cpu(op, xx, s).float()
            (g,) = torch.autograd.grad(y, xx, dy.float())
        return g.to(dy.dtype)
    x = x.contiguous()
    dy = dy.contiguous()
    dx = torch.empty_like(dy)
    _lib.check(_lib.lib().cgk_unary_backward(UNARY[op], _dt(x), x.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                             x.numel(), float(s), _lib.stream_ptr()), "cgk_unary_backward")
    _lib.count_launch()
    return dx


def binary(op: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Broadcasting a (op) b; both fp32 or both bf16."""
    shape = torch.broadcast_shapes(a.shape, b.shape)
    if not a.is_cuda:
        f = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div,
             "max": torch.maximum, "min": torch.minimum}[op]
        return f(a.float(), b.float()).to(a.dtype)
    out = torch.empty(shape, device=a.device, dtype=a.dtype)
    n = out.numel()
    L = _lib.lib()
    if tuple(a.shape) == tuple(b.shape) == tuple(shape) and a.is_contiguous() and b.is_contiguous():
        rc = L.cgk_binary(BINARY[op], _dt(a), a.data_ptr(), b.data_ptr(), out.data_ptr(), n, 0, None, None,
                          None, _lib.stream_ptr())
    else:
        nd = len(shape)
        if nd > 8:
            raise ValueError("binary: at most 8 dimensions")
        ae, be = a.expand(shape), b.expand(shape)
        sh = (ctypes.c_int * 8)(*shape, *([1] * (8 - nd)))
        sa = (ctypes.c_longlong * 8)(*ae.stride(), *([0] * (8 - nd)))
        sb = (ctypes.c_longlong * 8)(*be.stride(), *([0] * (8 - nd)))
        rc = L.cgk_binary(BINARY[op], _dt(a), a.data_ptr(), b.data_ptr(), out.data_ptr(), n, nd, sh, sa, sb,
                          _lib.stream_ptr())
    _lib.check(rc, "cgk_binary")
    _lib.count_launch()
    return out


REDUCE = {"sum": 0, "mean": 1, "max": 2, "min": 3}


def reduce(op: str, x: torch.Tensor, dim: int | None = None) -> torch.Tensor:
    """sum / mean / max / min over one axis or over everything; fp32 result."""
    if not x.is_cuda:
        xf = x.float()
        if dim is None:
            return {"sum": xf.sum, "mean": xf.mean, "max": xf.max, "min": xf.min}[op]().reshape(1)
        r = {"sum": xf.sum, "mean": xf.mean, "max": lambda d: xf.max(d).values,
             "min": lambda d: xf.min(d).values}[op](dim)
        return r
    x = x.contiguous()
    L = _lib.lib()
    if dim is None:
        out = torch.empty(1, device=x.device, dtype=torch.float32)
        scratch = _scratch(L.cgk_reduce_all_scratch_elems(x.numel()), x.device)
        _lib.check(L.cgk_reduce_all(REDUCE[op], _dt(x), x.data_ptr(), x.numel(), out.data_ptr(),
                                    scratch.data_ptr(), _lib.stream_ptr()), "cgk_reduce_all")
        _lib.count_launch(2)
        return out
    dim = dim % x.dim()
    outer = 1
    for s in x.shape[:dim]:
        outer *= s
    inner = 1
    for s in x.shape[dim + 1:]:
        inner *= s
    out = torch.empty(*x.shape[:dim], *x.shape[dim + 1:], device=x.device, dtype=torch.float32)
    _lib.check(L.cgk_reduce_axis(REDUCE[op], _dt(x), x.data_ptr(), out.data_ptr(), outer, x.shape[dim], inner,
                                 _lib.stream_ptr()), "cgk_reduce_axis")
    _lib.count_launch()
    return out


class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op):
        ctx.save_for_backward(x)
        ctx.op = op
        return unary(op, x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return unary_backward(ctx.op, x, dy), None


def activation(x, op: str):
    """relu / sigmoid / tanh / gelu / silu / exp / log / sqrt ... with autograd."""
    return _Act.apply(x, op)
