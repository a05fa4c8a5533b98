"""Convolutional classifier: (Conv2d 3x3 -> BatchNorm -> ReLU -> MaxPool 2x2) x len(channels) -> Flatten
-> Linear, trained with softmax cross-entropy; the model family behind the reference's Conv2D / MaxPool2D /
BatchNorm / Flatten layers (src/layers/conv2d.c:23-421, src/layers/activations.c:360-642), which the
reference ships without a model or an example that uses them.

On CUDA each convolution is an unfold kernel plus one tcgen05 GEMM (bias in its epilogue), pooling and
batch statistics run in the library's kernels and the classifier is a GEMM with the fused loss kernel
behind it; on CPU the same maths goes through PyTorch ops.
"""
from __future__ import annotations

import torch
from torch import nn

from ..nn.conv import BatchNorm, Conv2d, MaxPool2d
from ..nn.modules import Linear
from ..ops import loss as L


class ConvClassifier(nn.Module):
    def __init__(self, in_channels: int = 1, image: int = 28, channels=(16, 32), classes: int = 10, device=None, dtype=None):
        super().__init__()
        convs, norms = [], []
        c, side = in_channels, image
        for oc in channels:
            convs.append(Conv2d(c, oc, 3, stride=1, padding=1, bias=True, device=device, dtype=dtype))
            norms.append(BatchNorm(oc, device=device))
            c, side = oc, side // 2
        if side < 1:
            raise ValueError(f"image side {image} is too small for {len(channels)} pooling stages")
        self.convs, self.norms = nn.ModuleList(convs), nn.ModuleList(norms)
        self.pool = MaxPool2d(2)
        feat = c * side * side
        self.head = Linear(feat, classes, bias=True, init_std=(1.0 / feat) ** 0.5, device=device, dtype=dtype)

    def features(self, x):
        h = x.to(self.convs[0].weight.dtype)
        for conv, norm in zip(self.convs, self.norms):
            h = self.pool(torch.relu(norm(conv(h))))
        return h.flatten(1)

    def forward(self, x, targets=None, grad_scale=1.0):
        logits = self.head(self.features(x).to(self.head.weight.dtype))
        if targets is None:
            return logits
        return L.cross_entropy(logits, targets, grad_scale)
