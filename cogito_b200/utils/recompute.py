"""Activation recomputation: run a block without keeping its activations and run it a second
time, with autograd on, when its gradient is wanted.

``checkpoint(fn, *args)`` calls ``fn`` under ``no_grad`` and keeps only the arguments; its
backward restores the random-number state of the first run, re-runs ``fn`` on detached copies of
the tensor arguments with gradients enabled, back-propagates the incoming gradient through that
small graph and hands back the gradients of the arguments.  Parameters used inside ``fn`` get
their gradients the way they always do (``.grad`` or, for the kernels of this package, straight
into their ``main_grad`` buffer), so the block behaves as if nothing had been dropped, at the
price of one more forward pass per block and a peak of one block's activations.

Collectives inside ``fn`` (tensor-parallel blocks) are issued a second time during backward, by
every rank of the group alike, so they stay matched.

Reference counterpart: the ``use_recompute`` / ``activation_cache`` fields of cg_pipeline
(include/cg_pipeline.h:81-82), which nothing in the reference reads.
"""
from __future__ import annotations

import torch


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensors, *args):
        ctx.fn = fn
        ctx.rest = args[n_tensors:]
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
        tensors = args[:n_tensors]
        ctx.save_for_backward(*tensors)
        with torch.no_grad():
            out = fn(*tensors, *ctx.rest)
        return out

    @staticmethod
    def backward(ctx, *grads):
        tensors = [t.detach().requires_grad_(t.requires_grad) for t in ctx.saved_tensors]
        cpu_now = torch.get_rng_state()
        cuda_now = torch.cuda.get_rng_state() if ctx.cuda_rng is not None else None
        torch.set_rng_state(ctx.cpu_rng)
        if ctx.cuda_rng is not None:
            torch.cuda.set_rng_state(ctx.cuda_rng)
        try:
            with torch.enable_grad():
                out = ctx.fn(*tensors, *ctx.rest)
        finally:
            torch.set_rng_state(cpu_now)
            if cuda_now is not None:
                torch.cuda.set_rng_state(cuda_now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(t.grad if t.requires_grad else None for t in tensors) + (None,) * len(ctx.rest)


def checkpoint(fn, *args):
    """``fn(*args)`` with its activations dropped and recomputed in backward.  Tensor arguments must
    come first; the remaining arguments (shapes, flags, modules) are passed through unchanged."""
    n = 0
    while n < len(args) and torch.is_tensor(args[n]):
        n += 1
    if any(torch.is_tensor(a) for a in args[n:]):
        raise TypeError("checkpoint: tensor arguments must precede the others")
    if not torch.is_grad_enabled():
        return fn(*args)
    return _Checkpoint.apply(fn, n, *args)
