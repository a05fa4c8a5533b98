"""bf16 GEMM with fused epilogues on the tcgen05 tensor cores.

``gemm(a, b, ...)`` computes ``out[m, n] = epilogue(alpha * sum_k A(m, k) B(n, k))``
where each operand may be stored K-major or MN-major (see
``include/cogito_kernels.h``).  CUDA tensors run ``cgk_gemm_bf16``; CPU tensors
run an fp32 restatement of the same formula, which is also the oracle of the GPU
tests.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

ACT = {"none": 0, None: 0, "gelu": 1, "relu": 2, "silu": 3, "sigmoid": 4, "tanh": 5}

_default_max_ctas = 0


def set_default_max_ctas(n: int) -> None:
    """Caps the grid of every GEMM that does not name its own cap (0 = one CTA per SM).  A job whose
    point-to-point transfers run beside the compute kernels (pipeline parallelism) leaves a few SMs
    free this way: a persistent GEMM on every SM would keep the transfer kernels from starting."""
    global _default_max_ctas
    _default_max_ctas = max(0, int(n))


def default_max_ctas() -> int:
    return _default_max_ctas


def _act_cpu(name, x):
    if name in (None, "none"):
        return x
    if name == "gelu":
        return torch.nn.functional.gelu(x, approximate="tanh")
    if name == "relu":
        return torch.relu(x)
    if name == "silu":
        return torch.nn.functional.silu(x)
    if name == "sigmoid":
        return torch.sigmoid(x)
    if name == "tanh":
        return torch.tanh(x)
    raise ValueError(name)


def _dact_cpu(name, x):
    x = x.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        y = _act_cpu(name, x)
        (g,) = torch.autograd.grad(y.sum(), x)
    return g


def rope_reference(v, rope):
    """Rotary embedding of the first ``cols`` columns of v [M, N] (heads of D columns; row r is
    position r % T + pos0): the restatement of the GEMM's rotary epilogue."""
    cos, sin, cols, D, T, pos0, inverse = rope
    M_ = v.shape[0]
    pos = (torch.arange(M_, device=v.device) % T) + pos0
    c, s = cos.to(v.device)[pos].float(), sin.to(v.device)[pos].float() * (-1.0 if inverse else 1.0)     # [M, D/2]
    x = v[:, :cols].reshape(M_, cols // D, D)
    a, b = x[..., :D // 2], x[..., D // 2:]
    rot = torch.cat([a * c[:, None] - b * s[:, None], b * c[:, None] + a * s[:, None]], -1).reshape(M_, cols)
    return torch.cat([rot, v[:, cols:]], 1)


def gemm_reference(a, b, *, a_mn=False, b_mn=False, bias=None, act=None, residual=None,
                   aux_in=None, dact=None, alpha=1.0, accumulate_into=None, out_dtype=torch.bfloat16,
                   want_aux=False, rope=None):
    """fp32 restatement of the kernel's formula (any device)."""
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float() if b_mn else b.float().transpose(-1, -2)
    v = alpha * (A @ B)
    if bias is not None:
        v = v + bias.float()
    if rope is not None:
        v = rope_reference(v, rope)
    aux = v.to(a.dtype) if want_aux else None   # bf16 operands: the kernel stores the pre-activation in bf16
    v = _act_cpu(act, v)
    if aux_in is not None:
        v = v * _dact_cpu(dact, aux_in.float())
    if residual is not None:
        v = v + residual.float()
    if accumulate_into is not None:
        v = v + accumulate_into.float()
    out = v.to(out_dtype)
    return (out, aux) if want_aux else out


def fill_rope(g, rope, device) -> None:
    """Copies a rotary specification into a GemmArgs block (the tables must be fp32 on the device)."""
    cos, sin, cols, D, T, pos0, inverse = rope
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.device != device or not cos.is_contiguous() or not sin.is_contiguous():
        raise TypeError("rotary tables must be contiguous fp32 tensors on the operands' device")
    if cos.shape[-1] != D // 2 or cos.shape[0] < T + pos0:
        raise ValueError("rotary tables do not cover the positions asked for")
    g.rope_cos, g.rope_sin = cos.data_ptr(), sin.data_ptr()
    g.rope_cols, g.rope_D, g.rope_T, g.rope_pos0, g.rope_inverse = int(cols), int(D), int(T), int(pos0), int(bool(inverse))


def _ld(t: torch.Tensor) -> int:
    """Leading dimension of a 2-D (or batched 3-D) row-major view."""
    assert t.stride(-1) == 1, "innermost dimension must be contiguous"
    return t.stride(-2) if t.shape[-2] > 1 else max(t.shape[-1], t.stride(-2))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         bias: torch.Tensor | None = None, act: str | None = None,
         residual: torch.Tensor | None = None, aux_out: torch.Tensor | None = None,
         aux_in: torch.Tensor | None = None, dact: str | None = None,
         accumulate: bool = False, alpha: float = 1.0, force_simt: bool = False,
         max_ctas: int = 0, split_k: int = 0, rope=None) -> torch.Tensor:
    """``a``: [.., M, K] (or [.., K, M] when ``a_mn``); ``b``: [.., N, K] (or [.., K, N] when ``b_mn``).

    ``out`` may be given (bf16 or fp32; required for ``accumulate``).  ``aux_out``
    receives the pre-activation value in bf16.  ``aux_in`` / ``dact`` multiply the
    result by the activation derivative at ``aux_in``.  ``split_k`` (fp32 ``accumulate`` outputs
    only): 0 lets the launcher slice a long K range over idle SMs, 1 forbids it, n forces n slices.
    ``rope``: (cos, sin, cols, head_dim, T, pos0, inverse) applies the rotary embedding to the first
    ``cols`` output columns in the epilogue (2-D bf16 output, bias allowed, nothing else).
    """
    if a_mn:
        K, M = a.shape[-2], a.shape[-1]
    else:
        M, K = a.shape[-2], a.shape[-1]
    if b_mn:
        Kb, N = b.shape[-2], b.shape[-1]
    else:
        N, Kb = b.shape[-2], b.shape[-1]
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    batch_shape = a.shape[:-2]
    if b.shape[:-2] != batch_shape:
        raise ValueError("batch dimensions of a and b must match")
    batch = 1
    for s in batch_shape:
        batch *= s

    if not a.is_cuda:
        cpu_dtype = out_dtype if a.dtype == torch.bfloat16 else a.dtype   # fp32 in -> fp32 out on the host
        ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act=act, residual=residual,
                             aux_in=aux_in, dact=dact, alpha=alpha,
                             accumulate_into=out if accumulate else None,
                             out_dtype=out.dtype if out is not None else cpu_dtype,
                             want_aux=aux_out is not None, rope=rope)
        if aux_out is not None:
            ref, aux = ref
            aux_out.copy_(aux)
        if out is not None:
            out.copy_(ref)
            return out
        return ref

    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm: CUDA operands must be bf16")
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    if batch > 1:
        a = a.reshape(batch, *a.shape[-2:])
        b = b.reshape(batch, *b.shape[-2:])
        if a.stride(-1) != 1:
            a = a.contiguous()
        if b.stride(-1) != 1:
            b = b.contiguous()
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        out = torch.empty(*batch_shape, M, N, device=a.device, dtype=out_dtype)
    else:
        if out.shape[-2:] != (M, N) or out.stride(-1) != 1:
            raise ValueError(f"out has shape {tuple(out.shape)}, expected (.., {M}, {N}) row-major")
    out3 = out.reshape(batch, M, N) if batch > 1 else out
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm: out must be bf16 or fp32")

    g = _lib.GemmArgs()
    g.A, g.B, g.out = a.data_ptr(), b.data_ptr(), out3.data_ptr()
    g.M, g.N, g.K, g.batch = M, N, K, batch
    g.lda, g.ldb, g.ldc = _ld(a), _ld(b), _ld(out3)
    if batch > 1:
        g.strideA, g.strideB, g.strideC = a.stride(0), b.stride(0), out3.stride(0)
    else:
        g.strideA = g.strideB = g.strideC = 0
    g.a_mn, g.b_mn = int(a_mn), int(b_mn)
    g.out_fp32 = int(out.dtype == torch.float32)
    g.accumulate = int(accumulate)
    g.alpha = float(alpha)
    if bias is not None:
        if bias.numel() != N:
            raise ValueError("bias must have N elements")
        g.bias = bias.data_ptr()
        g.bias_fp32 = int(bias.dtype == torch.float32)
    g.act = ACT[act]
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape[-2:] == (M, N)
        g.residual, g.ldr = residual.data_ptr(), _ld(residual)
    if aux_out is not None:
        assert aux_out.dtype == torch.bfloat16 and aux_out.shape[-2:] == (M, N)
        g.aux_out, g.ldaux = aux_out.data_ptr(), _ld(aux_out)
    if aux_in is not None:
        assert aux_in.dtype == torch.bfloat16 and aux_in.shape[-2:] == (M, N)
        g.aux_in, g.ldauxin = aux_in.data_ptr(), _ld(aux_in)
        g.dact = ACT[dact]
    g.force_simt = int(force_simt)
    g.max_ctas = int(max_ctas) if max_ctas else _default_max_ctas
    g.split_k = int(split_k)
    if rope is not None:
        fill_rope(g, rope, a.device)
    _lib.check(_lib.lib().cgk_gemm_bf16(ctypes.byref(g), _lib.stream_ptr()), "cgk_gemm_bf16")
    _lib.count_launch()
    return out
