"""Fused data-parallel optimizer step against NCCL all-reduce + fused Adam.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        benchmarks/dp_step.py [--params 124] [--iters 10]

A flat parameter vector of ``--params`` million bf16 elements (GPT-2-small: 124) with fp32 gradients.
Timed with CUDA events on the launching stream, median over ``iters`` after warm-up, max over ranks:

* ``fused``: ``DPFusedAdam.step`` with every bucket still open (nothing overlapped with a backward
  pass): per bucket one kernel that sums the ranks' gradient parts over NVLink peer loads
  (reduce-scatter) and takes the sum of squares / overflow flag, then one kernel that exchanges the
  statistics, runs Adam on the owned parts and stores the new bf16 weights into every rank's copy.
* ``nccl``: ``all_reduce`` of the same fp32 gradient + ``FusedAdam.step`` (every rank updates all
  parameters), the unfused design.

``--device cpu`` runs the same two steps on gloo ranks with wall-clock time: a check of the script and
of the optimizer's host path, not a measurement.

One JSON line from rank 0 with both times, the bytes a rank receives over NVLink in the fused step
(fp32 gradient parts of the P - 1 peers' buckets it owns + the bf16 weights the peers broadcast) and the
fraction of the slower of that at 770 GB/s (measured) and the rank's HBM traffic at the measured copy rate.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--params", type=float, default=124.0, help="millions of parameters")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: gloo ranks and wall-clock time (checks the script and the optimizer's host path, not the kernels)")
    args = ap.parse_args()
    from cogito_b200.optim.fused import FusedAdam
    from cogito_b200.parallel.data_parallel import DPFusedAdam

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = args.device == "cuda"
    if cuda:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
    group = dist.group.WORLD
    n = int(args.params * 1e6) // (8 * world) * (8 * world)
    torch.manual_seed(0)

    def make():
        return [torch.nn.Parameter(torch.randn(n, device=dev, dtype=torch.bfloat16 if cuda else torch.float32) * 0.02)]

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.iters):
            if cuda:
                torch.cuda.synchronize()
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            else:
                import time
                dist.barrier()
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    fused = DPFusedAdam(make(), group, lr=1e-4)
    fused.grad.normal_()

    def step_fused():
        fused.step()
    ms_fused = timed(step_fused)
    buckets = fused.nbuckets
    del fused
    if cuda:
        torch.cuda.empty_cache()

    plain = FusedAdam(make(), lr=1e-4)
    plain.grad.normal_()

    def step_nccl():
        dist.all_reduce(plain.grad)
        plain.grad.div_(world)
        plain.step()
    ms_nccl = timed(step_nccl)

    P = world
    nvlink_in = (P - 1) / P * n * 4 + (P - 1) / P * n * 2           # gradient parts pulled + weights received
    hbm = n * 4 / P * P + n / P * (4 * 3 * 2) + n * 2                # own gradient parts read by the peers and here, Adam state r+w, weights written
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm_gbs = json.load(open(peaks))["hbm_gbs"] if os.path.exists(peaks) else 6650.0
    roof = max(nvlink_in / 770e9, hbm / (hbm_gbs * 1e9)) * 1e3
    if rank == 0:
        print(json.dumps({"case": "dp_step", "ranks": P, "params": n, "buckets": buckets, "fused_ms": round(ms_fused, 4),
                          "allreduce_plus_fused_adam_ms": round(ms_nccl, 4), "speedup": round(ms_nccl / ms_fused, 3),
                          "nvlink_MB_in_per_rank": round(nvlink_in / 1e6, 1), "roofline_ms": round(roof, 4),
                          "frac_of_roofline_measured": round(roof / ms_fused, 3)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
