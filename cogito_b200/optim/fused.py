"""Optimizers over flat buffers with a device-resident dynamic loss scaler.

All parameters of a model are re-pointed into one flat compute-dtype buffer; the
optimizer owns one flat fp32 master copy, one flat fp32 gradient buffer (each
parameter's ``main_grad`` is a view into it, filled by the backward GEMM
epilogues) and the flat state tensors.  A step is three launches — gradient
statistics, update, scaler update — with the skip-on-overflow decision taken on
the device, so no host synchronisation happens inside a training step.

Update rules and scaler constants follow the reference: Adam / AdamW
(src/optim/adam.c:10-46), SGD with momentum / Nesterov (src/optim/sgd.c:10-44),
loss scale 65536 in [1, 65536], x2 after 2000 clean steps, /2 and skip on overflow,
global-norm clip (src/core/bf16.c:88-94,115-198; src/optim/optimizer.c:66-88).
"""
from __future__ import annotations

import math

import torch

from ..ops import _lib


class FlatParams:
    """Flattens parameters into one buffer (padded per tensor to 16 bytes worth of
    elements) and keeps per-parameter views."""

    def __init__(self, params, align: int = 8, alloc=None, pad_to: int = 1):
        """alloc(nelems, dtype) -> 1-D tensor lets the caller place the flat buffer (for
        instance in symmetric memory); pad_to rounds the total length up."""
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        self.device = self.params[0].device
        self.dtype = self.params[0].dtype
        self.offsets = []
        off = 0
        for p in self.params:
            if p.device != self.device:
                raise ValueError("all parameters must live on one device")
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        self.total = (off + pad_to - 1) // pad_to * pad_to
        if alloc is not None:
            self.flat = alloc(self.total, self.dtype)
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.total, device=self.device, dtype=self.dtype)
        for p, o in zip(self.params, self.offsets):
            view = self.flat[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view

    def views(self, flat: torch.Tensor):
        return [flat[o:o + p.numel()].view(p.shape) for p, o in zip(self.params, self.offsets)]


class GradScaler:
    """Dynamic loss scale held in device memory (8 words: scale, good_steps,
    found_inf, step, skipped, norm_sq, pad, pad).  ``scale`` as a Python float is
    a host-side mirror that is only refreshed by :meth:`sync`."""

    def __init__(self, device, init_scale=65536.0, growth=2.0, backoff=0.5, window=2000,
                 min_scale=1.0, max_scale=65536.0, enabled=True):
        self.device = torch.device(device)
        self.enabled = enabled
        self.growth, self.backoff, self.window = growth, backoff, window
        self.min_scale, self.max_scale = min_scale, max_scale
        self.init_scale = init_scale if enabled else 1.0
        self.state = torch.zeros(8, device=self.device, dtype=torch.float32)
        self._host = {"scale": self.init_scale, "good_steps": 0, "found_inf": 0, "step": 0, "skipped": 0}
        if self.device.type == "cuda":
            _lib.check(_lib.lib().cgk_scaler_init(self.state.data_ptr(), float(self.init_scale),
                                                  _lib.stream_ptr()), "cgk_scaler_init")
            _lib.count_launch()

    # -- the device word holding the current scale (fp32), for kernels that read it
    @property
    def scale_tensor(self) -> torch.Tensor:
        return self.state[0:1]

    def sync(self) -> dict:
        """Copy the device state to the host (synchronises)."""
        if self.device.type == "cuda":
            raw = self.state.cpu()
            ints = raw.view(torch.int32)
            self._host = {"scale": float(raw[0]), "good_steps": int(ints[1]), "found_inf": int(ints[2]),
                          "step": int(ints[3]), "skipped": int(ints[4])}
        return dict(self._host)

    @property
    def scale(self) -> float:
        return self._host["scale"]

    def host_update(self, found_inf: bool) -> bool:
        """CPU path of the scaler rule; returns True when the step must be skipped."""
        h = self._host
        if found_inf:
            h["scale"] = max(h["scale"] * self.backoff, self.min_scale)
            h["good_steps"] = 0
            h["skipped"] += 1
            return True
        h["step"] += 1
        h["good_steps"] += 1
        if h["good_steps"] >= self.window:
            h["scale"] = min(h["scale"] * self.growth, self.max_scale)
            h["good_steps"] = 0
        return False

    def state_dict(self):
        return self.sync()

    def load_state_dict(self, d):
        self._host.update(d)
        if self.device.type == "cuda":
            raw = torch.zeros(8, dtype=torch.float32)
            ints = raw.view(torch.int32)
            raw[0] = d["scale"]
            ints[1], ints[2], ints[3], ints[4] = d["good_steps"], 0, d["step"], d["skipped"]
            self.state.copy_(raw)


class _FlatOptimizer:
    def __init__(self, params, lr, scaler: GradScaler | None, max_grad_norm: float, master_weights: bool):
        self.fp = FlatParams(list(params))
        self.lr = lr
        self.max_grad_norm = max_grad_norm
        dev = self.fp.device
        self.scaler = scaler if scaler is not None else GradScaler(dev, enabled=False)
        n = self.fp.total
        self.grad = torch.zeros(n, device=dev, dtype=torch.float32)
        low = self.fp.dtype != torch.float32
        self.master = self.fp.flat.float().clone() if (low and master_weights) else None
        if low and not master_weights:
            raise ValueError("low-precision parameters need fp32 master weights")
        for p, g in zip(self.fp.params, self.fp.views(self.grad)):
            p.main_grad = g
        # Model-parallel training: (overflow flag, sum of squares) of this rank's gradients -> the values of
        # the whole model replica.  A callable (found: tensor[1] int32, norm_sq: tensor[1] float32) -> None
        # that updates both in place (see parallel.llama_parallel.ModelParallelStats); None = local values.
        self.stats_sync = None
        self._scratch = None
        if dev.type == "cuda":
            ne = _lib.lib().cgk_grad_stats_scratch_elems(n)
            self._scratch = torch.empty(max(ne, 1), device=dev, dtype=torch.float32)

    @property
    def params(self):
        return self.fp.params

    def zero_grad(self):
        self.grad.zero_()
        for p in self.fp.params:
            p.grad = None

    def refresh_master(self):
        """Re-read the fp32 master copy from the parameters (after weights were loaded into them)."""
        if self.master is not None:
            self.master.copy_(self.fp.flat.float())

    def _gather_autograd_grads(self):
        """Parameters touched by ops that return ordinary gradients: fold .grad into main_grad."""
        for p in self.fp.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def _p32(self):
        return self.master if self.master is not None else self.fp.flat

    def _p16(self):
        return self.fp.flat if self.master is not None else None

    def _stats(self):
        _lib.check(_lib.lib().cgk_grad_stats(self.grad.data_ptr(), self.grad.numel(), self.scaler.state.data_ptr(),
                                             self._scratch.data_ptr(), 0, _lib.stream_ptr()), "cgk_grad_stats")
        _lib.count_launch(2)
        if self.stats_sync is not None:
            st = self.scaler.state
            self.stats_sync(st.view(torch.int32)[2:3], st[5:6])

    def _scaler_update(self):
        s = self.scaler
        _lib.check(_lib.lib().cgk_scaler_update(s.state.data_ptr(), float(s.growth if s.enabled else 1.0),
                                                float(s.backoff if s.enabled else 1.0), int(s.window),
                                                float(s.min_scale if s.enabled else 1.0),
                                                float(s.max_scale if s.enabled else 1.0), _lib.stream_ptr()),
                   "cgk_scaler_update")
        _lib.count_launch()

    # CPU helpers -------------------------------------------------------------
    def _cpu_prepare(self):
        """Returns (unscaled+clipped grad, skip)."""
        g = self.grad
        found = not bool(torch.isfinite(g).all())
        norm_sq = None
        if self.stats_sync is not None:
            f = torch.tensor([int(found)], dtype=torch.int32)
            n2 = (torch.nan_to_num(g, nan=0.0, posinf=0.0, neginf=0.0) ** 2).sum().reshape(1)
            self.stats_sync(f, n2)
            found, norm_sq = bool(f.item()), float(n2)
        # the gradients carry the scale the loss was multiplied with, i.e. the
        # value before this step's update of the scaler
        inv = 1.0 / self.scaler._host["scale"] if self.scaler.enabled else 1.0
        skip = self.scaler.host_update(found)
        if skip:
            return None, True
        g = g * inv
        if self.max_grad_norm > 0:
            norm = float(g.norm()) if norm_sq is None else math.sqrt(norm_sq) * inv
            if norm > self.max_grad_norm:
                g = g * (self.max_grad_norm / (norm + 1e-6))
        return g, False


class FusedAdam(_FlatOptimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 scaler: GradScaler | None = None, max_grad_norm: float = 0.0, master_weights: bool = True):
        super().__init__(params, lr, scaler, max_grad_norm, master_weights)
        self.beta1 = betas[0] if betas[0] > 0 else 0.9
        self.beta2 = betas[1] if betas[1] > 0 else 0.999
        self.eps = eps if eps > 0 else 1e-8
        self.weight_decay = weight_decay
        self.m = torch.zeros_like(self.grad)
        self.v = torch.zeros_like(self.grad)

    def step(self):
        self._gather_autograd_grads()
        if self.grad.is_cuda:
            self._stats()
            _lib.check(_lib.lib().cgk_adam_step(
                self._p32().data_ptr(), self.m.data_ptr(), self.v.data_ptr(), self.grad.data_ptr(),
                _lib.ptr(self._p16()), self.grad.numel(), float(self.lr), float(self.beta1), float(self.beta2),
                float(self.eps), float(self.weight_decay), float(self.max_grad_norm),
                self.scaler.state.data_ptr(), _lib.stream_ptr()), "cgk_adam_step")
            _lib.count_launch()
            self._scaler_update()
            return
        g, skip = self._cpu_prepare()
        if skip:
            return
        t = self.scaler._host["step"]
        p = self._p32()
        if self.weight_decay > 0:
            p.mul_(1.0 - self.lr * self.weight_decay)
        self.m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        self.v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1, bc2 = 1 - self.beta1 ** t, 1 - self.beta2 ** t
        p.sub_(self.lr * (self.m / bc1) / (torch.sqrt(self.v / bc2) + self.eps))
        if self.master is not None:
            self.fp.flat.copy_(p)

    def state_tensors(self):
        d = {"m": self.m, "v": self.v}
        if self.master is not None:
            d["master"] = self.master
        return d


class FusedSGD(_FlatOptimizer):
    def __init__(self, params, lr=0.01, momentum=0.0, weight_decay=0.0, nesterov=False,
                 scaler: GradScaler | None = None, max_grad_norm: float = 0.0, master_weights: bool = True):
        super().__init__(params, lr, scaler, max_grad_norm, master_weights)
        self.momentum, self.weight_decay, self.nesterov = momentum, weight_decay, nesterov
        self.vel = torch.zeros_like(self.grad) if momentum > 0 else None

    def step(self):
        self._gather_autograd_grads()
        if self.grad.is_cuda:
            self._stats()
            _lib.check(_lib.lib().cgk_sgd_step(
                self._p32().data_ptr(), _lib.ptr(self.vel), self.grad.data_ptr(), _lib.ptr(self._p16()),
                self.grad.numel(), float(self.lr), float(self.momentum), float(self.weight_decay),
                int(self.nesterov), float(self.max_grad_norm), self.scaler.state.data_ptr(),
                _lib.stream_ptr()), "cgk_sgd_step")
            _lib.count_launch()
            self._scaler_update()
            return
        g, skip = self._cpu_prepare()
        if skip:
            return
        p = self._p32()
        if self.weight_decay > 0:
            g = g + self.weight_decay * p
        if self.vel is not None:
            self.vel.mul_(self.momentum).add_(g)
            p.sub_(self.lr * (self.momentum * self.vel + g) if self.nesterov else self.lr * self.vel)
        else:
            p.sub_(self.lr * g)
        if self.master is not None:
            self.fp.flat.copy_(p)

    def state_tensors(self):
        d = {}
        if self.vel is not None:
            d["velocity"] = self.vel
        if self.master is not None:
            d["master"] = self.master
        return d


def step_lr(opt, step: int, step_size: int, gamma: float) -> None:
    """cg_optimizer_step_lr (src/optim/adam.c:113-117): multiply lr by gamma every step_size steps."""
    if step > 0 and step % step_size == 0:
        opt.lr *= gamma


def exp_lr(opt, initial_lr: float, gamma: float, t: int) -> None:
    """cg_optimizer_exp_lr (src/optim/adam.c:119-121): lr = initial * gamma^t."""
    opt.lr = initial_lr * math.pow(gamma, t)
