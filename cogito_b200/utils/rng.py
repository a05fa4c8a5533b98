"""Seeding.  Every layer draws its initial weights from a stream of its own,
derived from the global seed and the layer's construction index, so equal-shaped
layers start different (the reference seeds with 42 inside every constructor:
``srand(42)`` in src/layers/linear.c:213, ``cg_tensor_randn(..., 42, ...)`` in
src/layers/conv2d.c:292, which makes equal-shaped layers identical) and
a model's initial weights depend only on the seed and the construction order."""
from __future__ import annotations

import torch

_state = {"seed": None, "count": 0}


def manual_seed(seed: int) -> None:
    """Seed torch's global generator and restart the per-layer stream counter."""
    torch.manual_seed(seed)
    _state["seed"] = int(seed)
    _state["count"] = 0


def layer_generator(salt: int = 0) -> torch.Generator:
    """A CPU generator for the next constructed layer.  `salt` separates the streams of
    ranks that each build a different shard of the same layer (tensor parallelism)."""
    seed = torch.initial_seed()
    if _state["seed"] != seed:
        _state["seed"] = seed
        _state["count"] = 0
    _state["count"] += 1
    g = torch.Generator()
    g.manual_seed((seed * 1000003 + 7919 * _state["count"] + 104729 * salt) % (2 ** 63 - 1))
    return g


def uniform_(t: torch.Tensor, low: float, high: float, g: torch.Generator) -> torch.Tensor:
    with torch.no_grad():
        t.copy_((torch.rand(t.shape, generator=g) * (high - low) + low).to(t.dtype))
    return t


def normal_(t: torch.Tensor, std: float, g: torch.Generator) -> torch.Tensor:
    with torch.no_grad():
        t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))
    return t
