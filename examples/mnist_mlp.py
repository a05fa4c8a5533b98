"""MNIST-shaped classifier with the Python API: 784 -> 512 -> 512 -> 10, ReLU, fused softmax cross-entropy, Adam,
through the trainer (loss scaling, gradient clipping, JSON lines).  Synthetic separable digits unless the two idx
files are given.  Counterpart of examples/mnist.c.

    python examples/mnist_mlp.py [train-images-idx3-ubyte train-labels-idx1-ubyte] [--device cuda] [--epochs 3]

Under a launcher (`python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/mnist_mlp.py
--device cuda`) the ranks train data-parallel with the fused all-reduce + Adam kernels.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import cogito_b200 as cg  # noqa: E402
from cogito_b200.data.datasets import BatchIterator, load_mnist  # noqa: E402


def synthetic(n: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    proto = torch.randn(10, 784, generator=g)
    y = torch.randint(0, 10, (n,), generator=g)
    return 0.5 * proto[y] + 0.7 * torch.randn(n, 784, generator=g), y


def main(argv=None) -> float:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("files", nargs="*")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256, help="samples per rank and step")
    ap.add_argument("--samples", type=int, default=4096, help="synthetic samples per rank")
    args = ap.parse_args(argv)

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device(args.device, int(os.environ.get("LOCAL_RANK", "0"))) if args.device == "cuda" else torch.device("cpu")
    if world > 1:
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo")
    cg.manual_seed(0)
    model = cg.MLPClassifier(784, (512, 512), 10, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else None)
    scaler = cg.GradScaler(dev, enabled=dev.type == "cuda")
    if world > 1:
        parallel = cg.DataParallel(model, rank, world, dev)
        opt = parallel.make_optimizer(lr=1e-3, scaler=scaler)
    else:
        parallel, opt = None, cg.FusedAdam(model.parameters(), lr=1e-3, scaler=scaler, max_grad_norm=1.0)
    trainer = cg.Trainer(model, opt, parallel=parallel)
    x, y = load_mnist(*args.files[:2]) if len(args.files) >= 2 else synthetic(args.samples, seed=rank)
    x = x.reshape(x.shape[0], -1).float()
    last = float("nan")
    for epoch in range(args.epochs):
        total, hits, seen = 0.0, 0, 0
        for bx, by in BatchIterator(x, y, args.batch, shuffle=True, seed=epoch * world + rank):
            bx, by = bx.to(dev), by.to(dev)
            total += float(trainer.step(bx, by)) * by.numel()
            seen += by.numel()
        model.eval()
        with torch.no_grad():
            hits = int((model(x[:1024].to(dev)).argmax(-1).cpu() == y[:1024]).sum())
        model.train()
        last = total / max(seen, 1)
        if rank == 0:
            print(f"epoch {epoch + 1}  loss {last:.4f}  accuracy {hits / min(1024, len(y)):.3f}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return last


if __name__ == "__main__":
    main()
