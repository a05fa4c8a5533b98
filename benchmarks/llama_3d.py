"""Llama-7B-shaped 3-D parallel training step (the DP x TP x PP configuration of the baseline list).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        benchmarks/llama_3d.py [--dp 2 --tp 2 --pp 2] [--layers 32] [--seq 4096] [--microbatches 8] \\
        [--micro-batch 1] [--recompute block] [--steps 3] [--warmup 2]

Model: 32 layers, d_model 4096, 32 heads, d_ff 11008, vocabulary 32000 (random N(0, 0.02) weights,
uniform random token ids).  Each data-parallel replica runs ``microbatches`` micro-batches of
``micro-batch`` sequences through the 1F1B pipeline schedule, with dynamic loss scaling (2^16) and
gradient clipping on; the optimizer is the fused data-parallel Adam.  One JSON line from rank 0:
tokens/s over the whole job (device time of ``steps`` steps, max over ranks), ms per step, peak
memory per GPU, bytes sent between pipeline stages.  Weights are drawn on the device (the library's
default initialiser draws them on the host for reproducibility across device counts, which takes
minutes for 1.7 B parameters per rank and is not what this script measures).
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
    ap.add_argument("--dp", type=int, default=2)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--recompute", default="none", choices=["none", "block", "stage"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--d-ff", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: gloo ranks and wall-clock time with a small model (--d-model ...): a check of the script, not a measurement")
    args = ap.parse_args()

    from cogito_b200.models.llama import LlamaConfig
    from cogito_b200.ops import _lib
    from cogito_b200.parallel.groups import init_parallel
    from cogito_b200.parallel.llama_parallel import Trainer3D
    from cogito_b200.utils import rng

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.dp * args.tp * args.pp:
        raise SystemExit(f"world size {world} != dp*tp*pp = {args.dp * args.tp * args.pp}")
    cuda = args.device == "cuda"
    if cuda:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        torch.set_num_threads(1)
        dist.init_process_group("gloo")
    rng.manual_seed(0)

    def device_normal_(t, std, g):            # same signature as utils.rng.normal_; values are irrelevant here
        with torch.no_grad():
            return t.normal_(0.0, std)
    rng.normal_ = device_normal_
    torch.manual_seed(1234 + rank)
    cfg = LlamaConfig(vocab_size=args.vocab, d_model=args.d_model, n_head=args.heads, n_kv_head=args.heads, d_ff=args.d_ff,
                      n_layer=args.layers, max_seq_len=args.seq)
    ctx = init_parallel(args.dp, args.tp, args.pp)
    M, mb, T = args.microbatches, args.micro_batch, args.seq
    t3 = Trainer3D(cfg, ctx, dev, num_microbatches=M, micro_batch=mb, seq_len=T, lr=1e-4, loss_scale=65536.0,
                   max_grad_norm=1.0, recompute=None if args.recompute == "none" else args.recompute)
    g = torch.Generator().manual_seed(1 + ctx.coords.dp_rank)
    ids = torch.randint(0, cfg.vocab_size, (M * mb, T), generator=g).to(dev)
    tg = torch.randint(0, cfg.vocab_size, (M * mb, T), generator=g).to(dev)
    loss = None
    for _ in range(args.warmup):
        loss = t3.step(ids, tg)
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        torch.cuda.reset_peak_memory_stats(dev)
        _lib.reset_launches()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
    else:
        import time
        t0 = time.perf_counter()
    for _ in range(args.steps):
        loss = t3.step(ids, tg)
    if cuda:
        ev[1].record()
        torch.cuda.synchronize()
        elapsed, peak = ev[0].elapsed_time(ev[1]), torch.cuda.max_memory_allocated(dev) / 2 ** 30
    else:
        elapsed, peak = (time.perf_counter() - t0) * 1e3, 0.0
    t = torch.tensor([elapsed, peak, float(loss) if loss is not None else 0.0, 1.0 if loss is not None else 0.0], device=dev)
    mx = t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = t.clone()
    dist.all_reduce(sm)
    ms = float(mx[0]) / args.steps
    tokens = args.dp * M * mb * T
    if rank == 0:
        print(json.dumps({
            "metric": "train tok/s/box (Llama-7B shape, 3-D parallel)", "value": round(tokens / ms * 1e3, 1), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": round(ms, 2), "steps": args.steps, "warmup": args.warmup,
            "peak_mem_gib_per_gpu_max": round(float(mx[1]), 2), "loss": round(float(sm[2] / max(1.0, float(sm[3]))), 4),
            "launches_per_step_rank0": round(_lib.launches() / args.steps, 1) if cuda else None, "pipeline_p2p_bytes_rank0": t3.pipe.p2p_bytes,
            "optimizer": type(t3.opt).__name__, "scaler": t3.scaler.sync(),
            "config": {"layers": args.layers, "d_model": args.d_model, "heads": args.heads, "d_ff": args.d_ff, "vocab": args.vocab, "seq": T,
                       "microbatches": M, "micro_batch": mb, "dp": args.dp, "tp": args.tp, "pp": args.pp,
                       "schedule": "1F1B", "recompute": args.recompute, "dtype": "bf16" if cuda else "fp32", "data": "synthetic"}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
