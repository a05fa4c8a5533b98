"""Training loop front end: the call a user makes to run one optimizer step.

``Trainer.step(ids, targets)`` takes a global batch on the host (pinned) or on
the device, splits it into micro-batches, runs forward/backward with gradient
accumulation in the fp32 main-gradient buffer, applies the optimizer (with the
device-side overflow skip) and returns the mean loss as a device scalar.
No host synchronisation happens inside a step unless the caller reads the loss.
"""
from __future__ import annotations

import json
import time

import torch

from .optim.fused import FusedAdam, GradScaler


class Trainer:
    def __init__(self, model, optimizer, micro_batch: int | None = None, scaler: GradScaler | None = None,
                 log_path: str | None = None, parallel=None):
        self.model = model
        self.opt = optimizer
        self.micro_batch = micro_batch
        self.scaler = scaler if scaler is not None else optimizer.scaler
        self.device = optimizer.fp.device
        self.step_count = 0
        self.log_path = log_path
        self.parallel = parallel     # optional object with .reduce_gradients(opt) (data parallel)
        self._in_bufs = None

    def _stage(self, ids, targets):
        """Host tensors are copied through persistent device buffers on the current stream."""
        if ids.device == self.device:
            return ids, targets
        if self._in_bufs is None or self._in_bufs[0].shape != ids.shape:
            self._in_bufs = (torch.empty(ids.shape, dtype=ids.dtype, device=self.device),
                             torch.empty(targets.shape, dtype=targets.dtype, device=self.device))
        self._in_bufs[0].copy_(ids, non_blocking=True)
        self._in_bufs[1].copy_(targets, non_blocking=True)
        return self._in_bufs

    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        ids, targets = self._stage(ids, targets)
        B = ids.shape[0]
        mb = self.micro_batch or B
        n_micro = (B + mb - 1) // mb
        self.opt.zero_grad()
        total = None
        use_scale = self.scaler.enabled and self.device.type == "cuda"
        for i in range(n_micro):
            sl = slice(i * mb, min((i + 1) * mb, B))
            if use_scale:
                gs = self.scaler.scale_tensor * (1.0 / n_micro)
            elif self.scaler.enabled:
                gs = self.scaler.scale / n_micro
            else:
                gs = 1.0 / n_micro
            loss = self.model(ids[sl], targets[sl], grad_scale=gs)
            if i == n_micro - 1 and hasattr(self.opt, "arm"):
                self.opt.arm()           # last backward pass of the step: gradient buckets may leave as they fill
            loss.backward()
            d = loss.detach()
            total = d if total is None else total + d
        if self.parallel is not None:
            self.parallel.reduce_gradients(self.opt)
        self.opt.step()
        self.step_count += 1
        return total / n_micro

    def log(self, loss: float, tokens: int, ms: float) -> None:
        """Structured per-step record (JSON lines): step, loss, loss scale, skipped
        steps, tokens per second."""
        st = self.scaler.sync()
        rec = {"step": self.step_count, "loss": loss, "loss_scale": st["scale"], "skipped": st["skipped"],
               "tok_per_s": tokens / (ms * 1e-3) if ms > 0 else None, "time": time.time()}
        if self.log_path:
            with open(self.log_path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec
