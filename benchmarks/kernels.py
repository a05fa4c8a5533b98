"""Kernel micro-benchmarks with roofline fractions.

    python benchmarks/kernels.py <case> [--iters N] [--warmup W] [--small]

Cases: gemm, gemm_epilogue, flash_fwd, flash_bwd, layernorm, layernorm_bwd, rmsnorm, bias_grad,
cross_entropy, adam, int4_gemm, kv_attn, sample, all.  Each result is one JSON line: device time per call (CUDA events on the launching
stream, median of `iters` after `warmup` untimed calls, L2 flushed by writing a 256 MiB buffer
between calls), achieved TFLOP/s or GB/s, and the fraction of the measured peak taken from
MEASURED_PEAKS.json beside the repository root (copy bandwidth / cuBLAS bf16 burst) when that
file exists.  ``--small`` picks shapes a profiler can replay in seconds (a few GB at most, still
larger than L2 where DRAM figures matter).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

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
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, graph=False):
        """graph=True replays the call from a CUDA graph: for kernels of a few microseconds the
        Python wrapper is slower than the device, and the events would time the host."""
        for _ in range(self.warmup):
            fn()
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


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    t = Timer(args.iters, args.warmup)
    for name in (sorted(CASES) if args.case == "all" else [args.case]):
        CASES[name](t, args.small)
    from cogito_b200.ops import _lib
    code = _lib.read_status()[0]
    if code:
        raise SystemExit(f"device status {code}")


if __name__ == "__main__":
    main()
