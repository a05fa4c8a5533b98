"""Neural-network modules (torch.nn.Module subclasses) whose CUDA path runs the
sm_100a kernels.  Semantics follow the reference's layer set
(include/cg_layers.h, include/cg_transformer.h) with one autograd for everything.

Deliberate differences from the reference, each because the reference behaviour is
a defect: Linear weights are stored ``[out, in]`` (K-major for the tensor cores; the
reference stores ``[in, out]``, src/layers/linear.c:79-88); every layer gets its own
random stream (the reference reseeds with 42 in every constructor, :27-34, so
equal-shaped layers start identical).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import functional as F
from ..ops import loss as L
from ..ops import misc as M
from ..ops import norm as N
from ..utils import rng
from ..ops.attention import alibi_slopes, flash_attention, flash_attention_qkvpacked


def _maybe_bf16(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype != torch.bfloat16:
        return x.to(torch.bfloat16)
    return x


class Linear(nn.Module):
    """y = act(x W^T + b).  Xavier-uniform init like cg_linear_new (src/layers/linear.c:27-34)."""

    def __init__(self, in_features, out_features, bias=True, act=None, init_std=None,
                 device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.act = in_features, out_features, act
        w = torch.empty(out_features, in_features, device=device, dtype=dtype)
        g = rng.layer_generator()
        if init_std is None:
            limit = math.sqrt(6.0 / (in_features + out_features))
            rng.uniform_(w, -limit, limit, g)
        else:
            rng.normal_(w, init_std, g)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None

    def forward(self, x, residual=None):
        x = _maybe_bf16(x)
        return F.linear(x, self.weight, self.bias, self.act, residual)


class ReLU(nn.Module):
    def forward(self, x):
        return F.activation(x, "relu")


class Sigmoid(nn.Module):
    def forward(self, x):
        return F.activation(x, "sigmoid")


class Tanh(nn.Module):
    def forward(self, x):
        return F.activation(x, "tanh")


class GELU(nn.Module):
    """tanh approximation, constants 0.7978845608 / 0.044715 (src/cuda/tensor_kernels.c:179-188)."""

    def forward(self, x):
        return F.activation(x, "gelu")


class SiLU(nn.Module):
    def forward(self, x):
        return F.activation(x, "silu")


class Softmax(nn.Module):
    """Softmax over the last dimension (src/layers/activations.c:237-354)."""

    def forward(self, x):
        return torch.softmax(x.float(), -1).to(x.dtype)


class SwiGLU(nn.Module):
    def forward(self, x):
        return M.swiglu(x)


class Dropout(nn.Module):
    """Inverted dropout: kept values are scaled by 1/(1-p) in training, identity in eval."""

    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return M.dropout(x, self.p, self.training)


class Flatten(nn.Module):
    def forward(self, x):
        return x.reshape(x.shape[0], -1)


class LayerNorm(nn.Module):
    def __init__(self, dim, eps=1e-5, bias=True, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype)) if bias else None

    def forward(self, x, residual=None, passthrough=False):
        return N.layer_norm(_maybe_bf16(x), self.weight, self.bias, self.eps, residual, passthrough)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x, residual=None, passthrough=False):
        return N.rms_norm(_maybe_bf16(x), self.weight, self.eps, residual, passthrough)


class BatchNorm1d(nn.Module):
    """[B, F] batch norm with the reference's running-stat rule
    ``running = momentum * running + (1 - momentum) * batch`` (default momentum 0.1,
    src/layers/activations.c:496-499,618-619) and biased variance."""

    def __init__(self, features, eps=1e-5, momentum=0.1, device=None):
        super().__init__()
        self.eps, self.momentum = eps, momentum
        self.weight = nn.Parameter(torch.ones(features, device=device))
        self.bias = nn.Parameter(torch.zeros(features, device=device))
        self.register_buffer("running_mean", torch.zeros(features, device=device))
        self.register_buffer("running_var", torch.ones(features, device=device))

    def forward(self, x):
        xf = x.float()
        if self.training:
            mean = xf.mean(0)
            var = xf.var(0, unbiased=False)
            with torch.no_grad():
                self.running_mean.mul_(self.momentum).add_((1 - self.momentum) * mean)
                self.running_var.mul_(self.momentum).add_((1 - self.momentum) * var)
        else:
            mean, var = self.running_mean, self.running_var
        y = (xf - mean) * torch.rsqrt(var + self.eps) * self.weight.float() + self.bias.float()
        return y.to(x.dtype)


class Embedding(nn.Module):
    def __init__(self, num_embeddings, dim, init_std=0.02, device=None, dtype=None):
        super().__init__()
        w = torch.empty(num_embeddings, dim, device=device, dtype=dtype)
        self.weight = nn.Parameter(rng.normal_(w, init_std, rng.layer_generator()))

    def forward(self, ids, pos_weight=None):
        return M.embedding(ids, self.weight, pos_weight)


class Sequential(nn.Sequential):
    """cg_sequential: forward chains the layers; gradients flow through the one
    autograd tape, so ``loss.backward()`` reaches every parameter (the README
    snippet of the reference that its own library cannot train)."""

    def add(self, layer):
        self.append(layer)
        return self

    def num_params(self):
        return sum(p.numel() for p in self.parameters())

    def get_params(self):
        return list(self.parameters())
