#!/usr/bin/env python
"""Benchmark of the fused tensor-parallel kernels against their unfused twins.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/fused_tp.py [--config gpt2|llama|all] [--iters 20] [--sweep]

For each shape of the named configuration it checks the fused kernel against an fp32
restatement, then times (CUDA events on the launching stream, warm-up, maximum over ranks)

  * ``ag_gemm``  (all-gather -> GEMM, one kernel)  vs  NCCL all_gather_into_tensor + torch linear
  * ``gemm_rs``  (GEMM -> reduce-scatter, one kernel) vs torch.matmul + NCCL reduce_scatter_tensor

and prints one JSON line per case with: ms, bytes received over NVLink per rank, achieved
GB/s, FLOP, achieved TFLOP/s, the roofline time (the slower of FLOP at the measured cuBLAS
bf16 peak and NVLink bytes at the measured 770 GB/s per direction; the nominal 900 GB/s
figure is printed beside it) and the fraction of it that was reached.  Operands are larger
than the L2 at the GPT-2 shapes (201 MB activations and partial products).  The kernels use
the NVSwitch multicast path when the symmetric memory has one; ``COGITO_TP_NVLS=0`` times the
peer-load path instead.

``--sweep`` repeats the two GPT-2 layer shapes over several counts of copy / reduce CTAs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_MEASURED = 770e9      # peer copy, per direction per GPU, measured on this pool
NVLINK_NOMINAL = 900e9


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]) * 1e12, "measured"
    except Exception:
        return 1.59e15, "fallback"


def cases(config: str, P: int):
    out = []
    if config in ("gpt2", "all"):
        M, d, ff, V = 64 * 2048, 768, 3072, 50304
        out += [("gpt2 qkv", "ag", M, 3 * d // P // 8 * 8, d, None), ("gpt2 mlp-up", "ag", M, ff // P, d, "gelu"),
                ("gpt2 lm-head", "ag", M, V // P // 8 * 8, d, None),
                ("gpt2 attn-out", "rs", M, d, max(64, d // P // 64 * 64), None), ("gpt2 mlp-down", "rs", M, d, ff // P, None),
                ("gpt2 lm-head-bwd", "rs", M, d, V // P // 8 * 8, None)]
    if config in ("llama", "all"):
        M, d, ff = 4096, 4096, 11008
        kv = 1024
        out += [("llama qkv", "ag", M, (d + 2 * kv) // P, d, None), ("llama gate-up", "ag", M, 2 * ff // P // 8 * 8, d, None),
                ("llama o-proj", "rs", M, d, d // P, None), ("llama down", "rs", M, d, ff // P // 8 * 8, None)]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all", choices=["gpt2", "llama", "all"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--no-baseline", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)
    from cogito_b200.ops import _lib
    from cogito_b200.parallel.tp_ops import TPWorkspace, ag_gemm, gemm_rs

    P = world
    peak, peak_src = peaks()
    ws = TPWorkspace(dev, dist.group.WORLD if P > 1 else None, max_rows=64 * 2048, max_cols=4096 if args.config != "gpt2" else 768)
    if rank == 0:
        print(json.dumps({"ranks": P, "provider": ws.buf.provider if P > 1 else "local",
                          "multicast": bool(ws.nvls),
                          "bf16_peak_tflops": peak / 1e12, "peak_source": peak_src}), flush=True)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if P > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        if P > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def rel(a, b):
        return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()

    def report(name, kind, M, N, K, ms, base_ms, err, extra=None):
        flop = 2.0 * M * N * K
        link = (P - 1) / P * M * (K if kind == "ag" else N) * 2.0
        t_roof = max(flop / peak, link / NVLINK_MEASURED)
        rec = {"case": name, "kind": kind, "ranks": P, "M": M, "N": N, "K": K, "ms": round(ms, 4),
               "nvlink_MB_in_per_rank": round(link / 1e6, 1), "nvlink_GBps": round(link / ms / 1e6, 1),
               "tflops": round(flop / ms / 1e9, 1), "roofline_ms": round(t_roof * 1e3, 4),
               "bound": "compute" if flop / peak > link / NVLINK_MEASURED else "nvlink",
               "frac_of_roofline_measured": round(t_roof * 1e3 / ms, 3),
               "frac_of_roofline_nominal900": round(max(flop / peak, link / NVLINK_NOMINAL) * 1e3 / ms, 3),
               "nccl_cublas_ms": None if base_ms is None else round(base_ms, 4),
               "speedup_vs_nccl_cublas": None if base_ms is None else round(base_ms / ms, 3),
               "max_rel_err": err}
        if extra:
            rec.update(extra)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    ok = True
    for name, kind, M, N, K, act in cases(args.config, P):
        rows = M // P
        torch.manual_seed(7)
        if kind == "ag":
            xfull = torch.randn(M, K, device=dev, dtype=torch.bfloat16)          # same on all ranks (same seed)
            w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
            b = torch.randn(N, device=dev, dtype=torch.bfloat16)
            xs = xfull[rank * rows:(rank + 1) * rows].contiguous()
            out, gathered = ag_gemm(ws, xs, w, bias=b, act=act, keep=False)
            st = _lib.read_status()
            # check a slab of rows of every shard against fp32
            idx = torch.cat([torch.arange(r * rows, r * rows + 256, device=dev) for r in range(P)])
            ref = xfull[idx].float() @ w.float().T + b.float()
            if act == "gelu":
                ref = torch.nn.functional.gelu(ref, approximate="tanh")
            err = rel(out[idx], ref)
            good = err < 2e-2 and torch.equal(gathered, xfull) and st[0] == 0
            ok &= good
            del out, gathered, ref
            ms = timed(lambda: ag_gemm(ws, xs, w, bias=b, act=act, keep=False), args.iters)
            base = None
            if not args.no_baseline and P > 1:
                gath = torch.empty(M, K, device=dev, dtype=torch.bfloat16)

                def base_fn():
                    dist.all_gather_into_tensor(gath, xs)
                    y = torch.nn.functional.linear(gath, w, b)
                    return torch.nn.functional.gelu(y, approximate="tanh") if act == "gelu" else y
                base = timed(base_fn, args.iters)
                del gath
            report(name, kind, M, N, K, ms, base, err if good else f"FAILED {err} {st}")
            if args.sweep and name in ("gpt2 qkv", "gpt2 mlp-up") and P > 1:
                for nc in (4, 8, 16, 32):
                    ws.copy_ctas = nc
                    ms = timed(lambda: ag_gemm(ws, xs, w, bias=b, act=act, keep=False), args.iters)
                    report(name, kind, M, N, K, ms, base, None, {"copy_ctas": nc})
                ws.copy_ctas = 0
            del xfull, xs, w, b
        else:
            g = torch.Generator(device=dev).manual_seed(100 + rank)
            xr = torch.randn(M, K, device=dev, dtype=torch.bfloat16, generator=g)
            wr = torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
            b = torch.randn(N, device=dev, dtype=torch.bfloat16)
            res = torch.randn(rows, N, device=dev, dtype=torch.bfloat16)
            o = gemm_rs(ws, xr, wr, bias=b, residual=res)
            st = _lib.read_status()
            sl = slice(rank * rows, rank * rows + 512)
            part = torch.zeros(M if P > 1 else 512, N, device=dev, dtype=torch.float32)
            if P > 1:
                # the kernel ships bf16 partials; sum them in fp32 the same way
                part = torch.matmul(xr, wr.T).float()
                dist.all_reduce(part)
                ref = part[sl] + b.float() + res[:512].float()
            else:
                ref = xr[:512].float() @ wr.float().T + b.float() + res[:512].float()
            err = rel(o[:512], ref)
            good = err < 2e-2 and st[0] == 0
            ok &= good
            del part, ref, o
            ms = timed(lambda: gemm_rs(ws, xr, wr, bias=b, residual=res), args.iters)
            base = None
            if not args.no_baseline and P > 1:
                outp = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)

                def base_fn():
                    p = torch.matmul(xr, wr.T)
                    dist.reduce_scatter_tensor(outp, p)
                    return outp + b + res
                base = timed(base_fn, args.iters)
                del outp
            report(name, kind, M, N, K, ms, base, err if good else f"FAILED {err} {st}")
            if args.sweep and name in ("gpt2 attn-out", "gpt2 mlp-down") and P > 1:
                for nr in (8, 32, 64):
                    ws.reduce_ctas = nr
                    ms = timed(lambda: gemm_rs(ws, xr, wr, bias=b, residual=res), args.iters)
                    report(name, kind, M, N, K, ms, base, None, {"reduce_ctas": nr})
                ws.reduce_ctas = 0
            del xr, wr, b, res
        torch.cuda.empty_cache()
    st = _lib.read_status()
    print(f"[{rank}] ALL_OK {bool(ok)} status {st}", flush=True)
    if P > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if ok and st[0] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
