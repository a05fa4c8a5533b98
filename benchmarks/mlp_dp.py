"""Data-parallel MLP benchmark (the MNIST-shaped configuration of the baseline list).

    python benchmarks/mlp_dp.py [--steps 200] [--warmup 20] [--batch 256]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/mlp_dp.py

Model Linear(784, 512) -> ReLU -> Linear(512, 512) -> ReLU -> Linear(512, 10), cross-entropy, bf16 weights
with fp32 masters, dynamic loss scaling from 2^16, Adam lr 1e-3; synthetic inputs uniform in [0, 1) and
uniform labels, 256 samples per GPU and step (weak scaling).  With several GPUs the optimizer step is the
fused gradient all-reduce + unscale + Adam kernel over NVLink peer memory.  The step is a dozen small
kernels, so it is also timed as a CUDA-graph replay on one GPU (the multi-GPU step waits on peers inside
the kernel and is launched directly).  One JSON line from rank 0: samples/s over all GPUs, device time,
max over ranks.  The same configuration on PyTorch library code (DistributedDataParallel over NCCL,
bf16 autocast, torch.amp.GradScaler from 2^16, torch.optim.Adam) is timed in the same run and reported
under "baseline", with "vs_baseline" = value / baseline value.
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--batch", type=int, default=256, help="samples per GPU and step")
    args = ap.parse_args()

    from cogito_b200.models.mlp import MLPClassifier
    from cogito_b200.ops import _lib
    from cogito_b200.optim.fused import FusedAdam, GradScaler
    from cogito_b200.parallel.data_parallel import DataParallel
    from cogito_b200.train import Trainer
    from cogito_b200.utils import rng

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rng.manual_seed(0)
    model = MLPClassifier(784, (512, 512), 10, device=dev, dtype=torch.bfloat16)
    scaler = GradScaler(dev, init_scale=65536.0)
    parallel = None
    if world > 1:
        parallel = DataParallel(model, rank, world, dev)
        opt = parallel.make_optimizer(lr=1e-3, scaler=scaler)
    else:
        opt = FusedAdam(model.parameters(), lr=1e-3, scaler=scaler)
    trainer = Trainer(model, opt, parallel=parallel)
    g = torch.Generator().manual_seed(1 + rank)
    x = torch.rand(args.batch, 784, generator=g).to(dev)
    y = torch.randint(0, 10, (args.batch,), generator=g).to(dev)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    loss = [None]

    def step():
        loss[0] = trainer.step(x, y)

    for _ in range(max(3, args.warmup)):
        step()
    _lib.reset_launches()
    ms = timed(step, args.steps)
    launches = _lib.launches() / args.steps
    graph_ms = None
    if world == 1:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            graph_ms = timed(graph.replay, args.steps)
        except Exception as e:                          # the eager number above stands
            print(f"step not captured: {e!r}", file=sys.stderr)
    # ---- the same job on PyTorch library code ----
    base_ms = None
    try:
        tm = torch.nn.Sequential(torch.nn.Linear(784, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512), torch.nn.ReLU(),
                                 torch.nn.Linear(512, 10)).to(dev)
        ddp = torch.nn.parallel.DistributedDataParallel(tm, device_ids=[dev.index]) if world > 1 else tm
        topt = torch.optim.Adam(tm.parameters(), lr=1e-3, fused=True)
        tscaler = torch.amp.GradScaler("cuda", init_scale=65536.0)

        def tstep():
            topt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                l = torch.nn.functional.cross_entropy(ddp(x).float(), y)
            tscaler.scale(l).backward()
            tscaler.step(topt)
            tscaler.update()

        for _ in range(max(3, args.warmup)):
            tstep()
        base_ms = timed(tstep, args.steps)
    except Exception as e:
        print(f"baseline failed: {e!r}", file=sys.stderr)
    if rank == 0:
        best = min(ms, graph_ms) if graph_ms else ms
        print(json.dumps({
            "metric": "train samples/s/box (MNIST-shaped MLP, data parallel)", "value": round(world * args.batch / best * 1e3, 1),
            "unit": "samples/s", "n_gpus": world, "steps": args.steps, "ms_per_step": round(ms, 4),
            "ms_per_step_cuda_graph": None if graph_ms is None else round(graph_ms, 4), "scaling": "weak",
            "launches_per_step": launches, "loss": float(loss[0]), "loss_scale": scaler.sync()["scale"],
            "baseline": None if base_ms is None else {"impl": "torch DDP (NCCL) + autocast bf16 + GradScaler + fused Adam",
                                                      "value": round(world * args.batch / base_ms * 1e3, 1), "ms_per_step": round(base_ms, 4)},
            "vs_baseline": None if base_ms is None else round(base_ms / best, 3),
            "config": {"model": "784-512-512-10", "batch_per_gpu": args.batch, "dtype": "bf16", "optimizer": "adam 1e-3",
                       "loss_scale_init": 65536, "parallelism": f"dp{world}", "data": "synthetic"}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
