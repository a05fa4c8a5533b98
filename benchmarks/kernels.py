"""Kernel micro-benchmarks with roofline fractions.

    python benchmarks/kernels.py <case> [--iters N] [--warmup W] [--small]

Cases: gemm, gemm_epilogue, flash_fwd, flash_bwd, layernorm, layernorm_bwd, rmsnorm, bias_grad,
cross_entropy, adam, int4_gemm, kv_attn, sample, elementwise, jit_chain, reduce, rope, swiglu_dropout,
int4_quantize, spec_accept, all.  Each result is one JSON line: device time per call (CUDA events on the launching
stream, median of `iters` after `warmup` untimed calls, L2 flushed by writing a 256 MiB buffer
between calls), achieved TFLOP/s or GB/s, and the fraction of the measured peak taken from
MEASURED_PEAKS.json beside the repository root (copy bandwidth / cuBLAS bf16 burst) when that
file exists.  ``--small`` picks shapes a profiler can replay in seconds (a few GB at most, still
larger than L2 where DRAM figures matter).  Under ``all`` a case that raises is reported as an error
record and the others still run.  ``--device cpu`` runs the cases that have a host path (the last seven
of the list) with wall-clock time on tiny shapes: a check of the script, not a measurement.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

DEV = "cuda"

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, iters, warmup):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if DEV == "cuda" else None

    def __call__(self, fn, graph=False):
        """graph=True replays the call from a CUDA graph: for kernels of a few microseconds the
        Python wrapper is slower than the device, and the events would time the host."""
        for _ in range(self.warmup):
            fn()
        if DEV != "cuda":
            ts = []
            for _ in range(self.iters):
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
            ts.sort()
            return ts[len(ts) // 2]
        torch.cuda.synchronize()
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            fn = g.replay
            fn()
            torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]


def emit(name, ms, flops=None, bytes_=None, **extra):
    hbm, tf, src = peaks()
    rec = {"case": name, "ms": round(ms, 5), **extra}
    if flops:
        rec["tflops"] = round(flops / ms / 1e9, 1)
        rec[f"frac_of_{src}_bf16"] = round(flops / ms / 1e9 / tf, 3)
    if bytes_:
        rec["gbs"] = round(bytes_ / ms / 1e6, 1)
        rec[f"frac_of_{src}_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
    print(json.dumps(rec), flush=True)


def case_gemm(t, small):
    from cogito_b200.ops.gemm import gemm
    shapes = [(4096, 4096, 4096)] if small else [(8192, 8192, 8192), (16384, 3072, 768), (16384, 768, 3072), (16384, 50304, 768), (4096, 11008, 4096)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: gemm(a, b, out=out))
        # the library GEMM on the same operands, timed the same way (not under --small: the profiler's
        # kernel filter should see this library's kernel only)
        lib = None if small else t(lambda: torch.matmul(a, b.t(), out=out))
        extra = {} if lib is None else {"cublas_ms": round(lib, 5), "cublas_tflops": round(2.0 * M * N * K / lib / 1e9, 1),
                                        "vs_cublas": round(lib / ms, 3)}
        emit("gemm", ms, flops=2.0 * M * N * K, M=M, N=N, K=K, **extra)


def _qkv(B, T, H, Hk, D):
    mk = lambda h: torch.randn(B, T, h, D, device="cuda", dtype=torch.bfloat16)
    return mk(H), mk(Hk), mk(Hk)


def case_flash_fwd(t, small):
    from cogito_b200.ops.attention import flash_forward
    for B, T, H, Hk, D in ([(8, 2048, 12, 12, 64)] if small else [(8, 2048, 12, 12, 64), (4, 4096, 32, 8, 128)]):
        q, k, v = _qkv(B, T, H, Hk, D)
        emit("flash_fwd", t(lambda: flash_forward(q, k, v, causal=True)), flops=2.0 * B * H * T * T * D, B=B, T=T, H=H, Hk=Hk, D=D, causal=True)


def case_flash_bwd(t, small):
    from cogito_b200.ops.attention import flash_backward, flash_forward
    for B, T, H, Hk, D in ([(8, 2048, 12, 12, 64)] if small else [(8, 2048, 12, 12, 64), (4, 4096, 32, 8, 128)]):
        q, k, v = _qkv(B, T, H, Hk, D)
        o, lse = flash_forward(q, k, v, causal=True)
        do = torch.randn_like(o)
        emit("flash_bwd", t(lambda: flash_backward(do, q, k, v, o, lse, causal=True)), flops=5.0 * B * H * T * T * D, B=B, T=T, H=H, Hk=Hk, D=D, causal=True)


def _norm(t, small, rms):
    from cogito_b200.ops.norm import layer_norm, rms_norm
    R, C = (16384, 768) if not rms else (16384, 4096)
    if not small:
        R *= 4
    x = torch.randn(R, C, device="cuda", dtype=torch.bfloat16)
    g, b = torch.ones(C, device="cuda", dtype=torch.bfloat16), torch.zeros(C, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        ms = t((lambda: rms_norm(x, g)) if rms else (lambda: layer_norm(x, g, b)))
    emit("rmsnorm" if rms else "layernorm", ms, bytes_=2.0 * R * C * 2, rows=R, cols=C)


def case_layernorm(t, small):
    _norm(t, small, False)


def case_layernorm_bwd(t, small):
    """Backward of the residual-stream LayerNorm: reads x, dy and the second gradient of the
    residual stream, writes dx (4 passes over [rows, cols]) plus the small dgamma / dbeta."""
    from cogito_b200.ops.norm import layer_norm
    R, C = (16384 if small else 131072), 768
    x = torch.randn(R, C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.ones(C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer_norm(x, g, b)
    dy = torch.randn_like(y)

    def bwd():
        x.grad = g.grad = b.grad = None
        y.backward(dy, retain_graph=True)
    emit("layernorm_bwd", t(bwd), bytes_=3.0 * R * C * 2, rows=R, cols=C)


def case_bias_grad(t, small):
    """Column sums of a [rows, cols] bf16 gradient (the bias gradient of a linear layer)."""
    from cogito_b200.ops.functional import colsum
    R = 16384 if small else 131072
    for C in (768, 3072):
        dy = torch.randn(R, C, device="cuda", dtype=torch.bfloat16)
        emit("bias_grad", t(lambda: colsum(dy)), bytes_=1.0 * R * C * 2, rows=R, cols=C)


def case_gemm_epilogue(t, small):
    """The GPT-2 block's K = 768 projections with their epilogues (bias, GELU with the pre-activation
    kept for backward, residual add, activation derivative)."""
    from cogito_b200.ops.gemm import gemm
    M = 16384 if small else 65536
    x = torch.randn(M, 768, device="cuda", dtype=torch.bfloat16)
    w_up = torch.randn(3072, 768, device="cuda", dtype=torch.bfloat16) * 0.02
    w_dn = torch.randn(768, 3072, device="cuda", dtype=torch.bfloat16) * 0.02      # [out, in]: the dgrad reads it as [K, N]
    w_pr = torch.randn(768, 768, device="cuda", dtype=torch.bfloat16) * 0.02
    w_qkv = torch.randn(2304, 768, device="cuda", dtype=torch.bfloat16) * 0.02
    b_up = torch.zeros(3072, device="cuda", dtype=torch.bfloat16)
    b_pr = torch.zeros(768, device="cuda", dtype=torch.bfloat16)
    b_qkv = torch.zeros(2304, device="cuda", dtype=torch.bfloat16)
    aux = torch.empty(M, 3072, device="cuda", dtype=torch.bfloat16)
    out_up = torch.empty(M, 3072, device="cuda", dtype=torch.bfloat16)
    cases = [
        ("qkv: bias", lambda: gemm(x, w_qkv, bias=b_qkv), 2304, 768),
        ("proj: bias + residual", lambda: gemm(x, w_pr, bias=b_pr, residual=x), 768, 768),
        ("mlp up: bias + gelu, pre-activation kept", lambda: gemm(x, w_up, bias=b_up, act="gelu", aux_out=aux, out=out_up), 3072, 768),
        ("mlp down dgrad: x gelu'(pre-activation)", lambda: gemm(x, w_dn, b_mn=True, aux_in=aux, dact="gelu", out=out_up), 3072, 768),
    ]
    for name, fn, N, K in cases:
        emit("gemm_epilogue", t(fn), flops=2.0 * M * N * K, what=name, M=M, N=N, K=K)


def case_rmsnorm(t, small):
    _norm(t, small, True)


def case_cross_entropy(t, small):
    from cogito_b200.ops.loss import cross_entropy
    R, V = (4096 if small else 16384), 50304
    logits = torch.randn(R, V, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    tg = torch.randint(0, V, (R,), device="cuda")

    def fwd_bwd():
        logits.grad = None
        cross_entropy(logits, tg).backward()
    emit("cross_entropy_fwd_bwd", t(fwd_bwd), bytes_=2.0 * R * V * 2, rows=R, vocab=V)


def case_adam(t, small):
    from cogito_b200.optim.fused import FusedAdam
    n = (32 if small else 124) * 1024 * 1024
    p = torch.nn.Parameter(torch.zeros(n, device="cuda", dtype=torch.bfloat16))
    opt = FusedAdam([p], lr=1e-3)
    opt.grad.normal_()
    emit("adam_step", t(opt.step), bytes_=n * (4 + 4 * 2 * 3 + 2.0), elements=n)      # grad r, master/m/v r+w, bf16 w


def case_int4_gemm(t, small):
    from cogito_b200.quant.int4 import Int4Linear
    for M, K, N in ([(16, 4096, 32000)] if small else [(16, 4096, 4096), (80, 4096, 11008), (80, 11008, 4096), (16, 4096, 32000)]):
        lin = Int4Linear(torch.randn(N, K, device="cuda") * 0.02, None, 128)
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        emit("int4_gemm", t(lambda: lin(x), graph=True), kernel=lin.kernel, bytes_=K * N / 2 + K * N / 128 * 4, flops=2.0 * M * N * K, M=M, N=N, K=K)


def case_kv_attn(t, small):
    from cogito_b200.serve.kv_cache import PagedKVCacheInt4
    B, hist, Tq = (4 if small else 16), 2048, 5
    c = PagedKVCacheInt4(1, B, hist + 64, 8, 128, 32, 64, "cuda")
    mk = lambda T, h: torch.randn(B, T, h, 128, device="cuda", dtype=torch.bfloat16)
    c.append(0, mk(hist, 8), mk(hist, 8))
    c.commit(hist)
    c.append(0, mk(Tq, 8), mk(Tq, 8))
    q = mk(Tq, 32)
    emit("kv_int4_attention", t(lambda: c.attention(0, q), graph=True), bytes_=B * hist * 8 * (128 + 2 * 16.0), B=B, history=hist, Tq=Tq)


def case_sample(t, small):
    from cogito_b200.serve.sampling import sample
    rows, V = (16 if small else 80), 32000
    lg = torch.randn(rows, V, device="cuda")
    step = torch.zeros(1, dtype=torch.int64, device="cuda")
    emit("sample_topk_topp", t(lambda: sample(lg, 0.8, 50, 0.9, 1, step, return_probs=True), graph=True), bytes_=rows * V * 8.0, rows=rows, vocab=V)


def _n(small, big, little):
    """Element count: `big` for a measurement, `little` under --small, a few thousand on the host."""
    return 4096 if DEV != "cuda" else (little if small else big)


def case_elementwise(t, small):
    """One unary and one broadcasting binary kernel of the elementwise library (bf16, 2 bytes in and out per element)."""
    from cogito_b200.ops.functional import binary, unary
    n = _n(small, 256 << 20, 64 << 20)
    x = torch.randn(n // 1024, 1024, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(1024, device=DEV, dtype=torch.bfloat16)
    emit("elementwise", t(lambda: unary("gelu", x)), bytes_=2.0 * n * 2, what="gelu", elements=n)
    emit("elementwise", t(lambda: binary("add", x, b)), bytes_=2.0 * n * 2, what="add, row broadcast", elements=n)


def case_jit_chain(t, small):
    """A chain the tracer fuses into one generated kernel: sigmoid(a * b + c) * a, three inputs, one output."""
    from cogito_b200.jit.fuse import fuse, sigmoid
    n = _n(small, 128 << 20, 32 << 20)
    a, b, c = (torch.randn(n, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    f = fuse(lambda a, b, c: sigmoid(a * b + c) * a)
    f(a, b, c)                                                         # trace + compile outside the timed calls
    emit("jit_chain", t(lambda: f(a, b, c)), bytes_=4.0 * n * 2, elements=n)


def case_reduce(t, small):
    """Sum over everything and over the rows of a [rows, 1024] bf16 matrix."""
    from cogito_b200.ops.functional import reduce
    n = _n(small, 256 << 20, 64 << 20)
    x = torch.randn(n // 1024, 1024, device=DEV, dtype=torch.bfloat16)
    emit("reduce", t(lambda: reduce("sum", x)), bytes_=1.0 * n * 2, what="sum, all", elements=n)
    emit("reduce", t(lambda: reduce("sum", x, 1)), bytes_=1.0 * n * 2, what="sum, last axis", elements=n)
    emit("reduce", t(lambda: reduce("max", x, 0)), bytes_=1.0 * n * 2, what="max, first axis", elements=n)


def case_rope(t, small):
    """Rotary embedding in place on [B, T, H, D] bf16 (one read and one write of the tensor)."""
    from cogito_b200.ops.misc import rope_apply_, rope_tables
    B, T, H, D = (2, 64, 2, 64) if DEV != "cuda" else ((4, 4096, 32, 128) if not small else (2, 2048, 32, 128))
    x = torch.randn(B, T, H, D, device=DEV, dtype=torch.bfloat16)
    cos_t, sin_t = rope_tables(T, D, device=DEV)
    emit("rope", t(lambda: rope_apply_(x, cos_t, sin_t)), bytes_=2.0 * x.numel() * 2, B=B, T=T, H=H, D=D)


def case_swiglu_dropout(t, small):
    """SwiGLU split ([rows, 2F] -> [rows, F]) and dropout (counter-based mask) on bf16."""
    from cogito_b200.ops.misc import dropout, swiglu
    rows, F = (64, 128) if DEV != "cuda" else ((16384, 11008) if not small else (4096, 11008))
    x = torch.randn(rows, 2 * F, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        emit("swiglu", t(lambda: swiglu(x)), bytes_=3.0 * rows * F * 2, rows=rows, features=F)
        h = torch.randn(rows, F, device=DEV, dtype=torch.bfloat16)
        emit("dropout", t(lambda: dropout(h, 0.1, True, seed=1)), bytes_=2.0 * rows * F * 2, rows=rows, features=F)


def case_int4_quantize(t, small):
    """Flat groups of 128: quantise an fp32 tensor (4 bytes in, ~0.53 out per element) and dequantise it to bf16."""
    from cogito_b200.quant.int4 import dequantize_int4, quantize_int4
    n = _n(small, 128 << 20, 32 << 20)
    x = torch.randn(n, device=DEV)
    packed, scales = quantize_int4(x, 128)
    emit("int4_quantize", t(lambda: quantize_int4(x, 128)), bytes_=n * (4 + 0.5 + 4 / 128), elements=n)
    emit("int4_dequantize", t(lambda: dequantize_int4(packed, scales, n, 128, torch.bfloat16)), bytes_=n * (0.5 + 4 / 128 + 2), elements=n)


def case_spec_accept(t, small):
    """Accept / correct / commit for 16 sequences, gamma 4, vocabulary 32000 (latency-bound), and the tree mask."""
    from cogito_b200.serve.sampling import spec_accept, tree_attention_mask
    B, g, V = (2, 4, 512) if DEV != "cuda" else (16, 4, 32000)
    q = torch.softmax(torch.randn(B, g, V, device=DEV), -1)
    p = torch.softmax(torch.randn(B, g + 1, V, device=DEV), -1)
    tok = torch.randint(0, V, (B, g), device=DEV, dtype=torch.int32)
    step = torch.zeros(1, dtype=torch.int64, device=DEV) if DEV == "cuda" else 0
    emit("spec_accept", t(lambda: spec_accept(tok, q, p, 1, step), graph=DEV == "cuda"), bytes_=(2 * g + 1) * B * V * 4.0, B=B, gamma=g, vocab=V)
    parents = torch.tensor([-1, 0, 0, 1, 1, 2, 2, 3], dtype=torch.int32, device=DEV)
    emit("tree_mask", t(lambda: tree_attention_mask(parents, 512), graph=DEV == "cuda"), bytes_=4.0 * (512 + 8) ** 2, prefix=512, nodes=8)


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}
HOST_CASES = ("elementwise", "jit_chain", "reduce", "rope", "swiglu_dropout", "int4_quantize", "spec_accept")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    args = ap.parse_args()
    global DEV
    DEV = args.device
    if DEV == "cpu" and args.case != "all" and args.case not in HOST_CASES:
        raise SystemExit(f"{args.case} has no host path; with --device cpu choose one of {', '.join(HOST_CASES)} or all")
    t = Timer(args.iters, args.warmup)
    names = [n for n in sorted(CASES) if DEV == "cuda" or n in HOST_CASES] if args.case == "all" else [args.case]
    for name in names:
        if args.case != "all":
            CASES[name](t, args.small)
            continue
        try:
            CASES[name](t, args.small)
        except Exception as e:                               # one broken case must not hide the others' numbers
            print(json.dumps({"case": name, "error": repr(e)[:300]}), flush=True)
    if DEV == "cuda":
        from cogito_b200.ops import _lib
        code = _lib.read_status()[0]
        if code:
            raise SystemExit(f"device status {code}")


if __name__ == "__main__":
    main()
