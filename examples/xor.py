"""XOR with the Python API: Linear(2,4) -> ReLU -> Linear(4,1) -> Sigmoid, MSE, SGD lr 0.5 momentum 0.9, 5000
full-batch epochs, seed 0.  Counterpart of examples/xor.c (the C API) and of the reference's examples/xor.c.

    python examples/xor.py [epochs] [cpu|cuda]
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import cogito_b200 as cg  # noqa: E402
from cogito_b200.ops import loss as L  # noqa: E402


def main(epochs: int = 5000, device: str = "cpu") -> float:
    cg.manual_seed(0)
    net = cg.nn.Sequential(cg.nn.Linear(2, 4, device=device), cg.nn.ReLU(), cg.nn.Linear(4, 1, device=device), cg.nn.Sigmoid())
    opt = cg.FusedSGD(net.parameters(), lr=0.5, momentum=0.9, master_weights=False)
    x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]], device=device)
    y = torch.tensor([[0.], [1.], [1.], [0.]], device=device)
    loss = None
    for epoch in range(epochs):
        opt.zero_grad()
        loss = L.mse_loss(net(x), y)
        loss.backward()
        opt.step()
        if epoch % 1000 == 0:
            print(f"epoch {epoch} loss {float(loss.detach()):.6f}")
    for row, out in zip(x.tolist(), net(x).flatten().tolist()):
        print(f"{row[0]:g} xor {row[1]:g} -> {out:.4f}")
    print(f"final loss {float(loss.detach()):.6f}")
    return float(loss.detach())


if __name__ == "__main__":
    final = main(int(sys.argv[1]) if len(sys.argv) > 1 else 5000, sys.argv[2] if len(sys.argv) > 2 else "cpu")
    sys.exit(0 if final < 0.01 else 1)
