"""MLP classifier: Linear -> ReLU -> ... -> Linear with cross-entropy, the MNIST-shaped
data-parallel workload (784 -> 512 -> 512 -> 10) and the XOR network (2 -> 4 -> 1 with a
sigmoid and MSE).  Reference: examples/mnist.c, examples/xor.c.

On CUDA every Linear + activation is one tcgen05 GEMM with the bias and activation in its
epilogue; the loss is the fused softmax-cross-entropy kernel.
"""
from __future__ import annotations

import torch
from torch import nn

from ..nn.modules import Linear
from ..ops import loss as L


class MLPClassifier(nn.Module):
    def __init__(self, in_features: int = 784, hidden=(512, 512), classes: int = 10, device=None, dtype=None):
        super().__init__()
        dims = [in_features, *hidden, classes]
        n = len(dims) - 1
        self.layers = nn.ModuleList([Linear(a, b, bias=True, act="relu" if i < n - 1 else None, init_std=(2.0 / a) ** 0.5,
                                            device=device, dtype=dtype)
                                     for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))])

    def forward(self, x, targets=None, grad_scale=1.0):
        h = x.to(self.layers[0].weight.dtype)
        for lin in self.layers:
            h = lin(h)
        if targets is None:
            return h
        return L.cross_entropy(h, targets, grad_scale)


class XorNet(nn.Module):
    """Linear(2,4) -> ReLU -> Linear(4,1) -> Sigmoid (Xavier-uniform weights)."""

    def __init__(self, device=None):
        super().__init__()
        self.l1 = Linear(2, 4, bias=True, act="relu", device=device)
        self.l2 = Linear(4, 1, bias=True, act="sigmoid", device=device)

    def forward(self, x):
        return self.l2(self.l1(x))
