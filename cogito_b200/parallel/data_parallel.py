"""Data parallelism whose optimizer step is one fused kernel: gradient all-reduce over
NVLink peer memory + loss-scale unscale / overflow check + global-norm clip + Adam +
broadcast of the new weights (``cgk_dp_adam_step``, csrc/comm/dp_adam.cu).

Each rank keeps the fp32 master weights and Adam moments of one slice of the flat
parameter space only (sharded optimizer state); parameters and gradients live in
symmetric memory so that peers can read gradients and write updated weights.

On CPU ranks (gloo) the same step is an all-reduce followed by the local update rule,
which is the oracle of the GPU test.

Reference counterparts: PARALLEL_DATA / dp_group / cg_pipeline_allreduce_grads
(include/cg_pipeline.h:16,72,113 — declared only).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int32, c_int64, c_uint32, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..optim.fused import FlatParams, GradScaler
from .symm import SymmetricBuffer


class DpAdamArgs(Structure):
    _fields_ = [("rank", c_int32), ("ranks", c_int32), ("epoch", c_int32), ("grid_ctas", c_int32),
                ("grad_ptrs", c_void_p * 8), ("param_lp_ptrs", c_void_p * 8), ("param_fp_ptrs", c_void_p * 8),
                ("signal_ptrs", c_void_p * 8),
                ("master", c_void_p), ("m", c_void_p), ("v", c_void_p), ("gsum", c_void_p),
                ("begin", c_int64), ("count", c_int64),
                ("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float),
                ("weight_decay", c_float), ("max_grad_norm", c_float), ("grad_mul", c_float),
                ("growth", c_float), ("backoff", c_float), ("min_scale", c_float), ("max_scale", c_float),
                ("window", c_int32), ("scaler", c_void_p), ("block_part", c_void_p), ("grid_bar", c_void_p),
                ("grid_bar_base", c_uint32)]


class DPFusedAdam:
    """Adam over a data-parallel group.  Same surface as ``FusedAdam`` (``fp``, ``grad``,
    ``scaler``, ``zero_grad``, ``step``); gradients are summed over the group inside ``step``
    (use ``average=True`` to divide by the group size)."""

    def __init__(self, params, group=None, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 scaler: GradScaler | None = None, max_grad_norm: float = 0.0, average: bool = True):
        params = [p for p in params if p.requires_grad]
        self.group = group
        self.ranks = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        P = self.ranks
        dev = params[0].device
        self.cuda = dev.type == "cuda"
        self.lr, self.beta1, self.beta2, self.eps = lr, betas[0], betas[1], eps
        self.weight_decay, self.max_grad_norm, self.average = weight_decay, max_grad_norm, average
        self.scaler = scaler if scaler is not None else GradScaler(dev, enabled=False)
        esize = params[0].element_size()
        n_guess = sum((p.numel() + 7) // 8 * 8 for p in params)
        n = (n_guess + 4 * P - 1) // (4 * P) * (4 * P)
        self.n = n
        self.low = params[0].dtype != torch.float32
        if self.cuda:
            p_bytes = (n * esize + 255) // 256 * 256
            g_bytes = (n * 4 + 255) // 256 * 256
            self.sym = SymmetricBuffer(p_bytes + g_bytes + 256, dev, group)
            self._p_off, self._g_off, self._s_off = 0, p_bytes, p_bytes + g_bytes
            alloc = lambda ne, dt: self.sym.view(0, (ne,), dt)
            self.fp = FlatParams(params, alloc=alloc, pad_to=4 * P)
            assert self.fp.total == n
            self.grad = self.sym.view(self._g_off, (n,), torch.float32)
        else:
            self.fp = FlatParams(params, pad_to=4 * P)
            self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        for p, g in zip(self.fp.params, self.fp.views(self.grad)):
            p.main_grad = g
        per = n // P
        self.begin, self.count = self.rank * per, per
        sl = slice(self.begin, self.begin + self.count)
        self.master = self.fp.flat[sl].float().clone() if self.low else None
        self.m = torch.zeros(per, dtype=torch.float32, device=dev)
        self.v = torch.zeros(per, dtype=torch.float32, device=dev)
        self.epoch = 0
        if self.cuda:
            L = _lib.lib()
            L.cgk_dp_adam_step.argtypes = [POINTER(DpAdamArgs), c_void_p]
            self.grid = min(L.cgk_dp_adam_max_ctas(), max(1, (per // 4 + 255) // 256))
            self.gsum = torch.empty(per, dtype=torch.float32, device=dev)
            self.block_part = torch.zeros(2 * self.grid, dtype=torch.float32, device=dev)
            self.grid_bar = torch.zeros(1, dtype=torch.int32, device=dev)
            self.calls = 0

    @property
    def params(self):
        return self.fp.params

    def zero_grad(self):
        self.grad.zero_()
        for p in self.fp.params:
            p.grad = None

    def refresh_master(self):
        """Re-read this rank's fp32 master slice from the parameters (after a weight load)."""
        if self.master is not None:
            self.master.copy_(self.fp.flat[self.begin:self.begin + self.count].float())

    # -- checkpoint / elastic restart ------------------------------------------------------
    def state_tensors(self):
        """This rank's shard of the optimizer state."""
        d = {"m": self.m, "v": self.v}
        if self.master is not None:
            d["master"] = self.master
        return d

    def shard_state(self) -> dict:
        """Everything a restart needs from this rank: its shard, where the shard sits in the flat
        parameter vector, and the step / loss-scale state (host copies)."""
        d = {k: v.detach().cpu().clone() for k, v in self.state_tensors().items()}
        d.update(begin=self.begin, count=self.count, n=self.n, ranks=self.ranks, scaler=self.scaler.state_dict())
        return d

    def load_resharded(self, shards) -> None:
        """Restore from the shards of a run with ANY data-parallel size (a rank was lost, or ranks
        were added).  Parameters start at the same offsets of the flat vector whatever the group
        size (only the padding at its end depends on it), so this rank's slice is filled from the
        overlap with each old shard; positions no old shard covers are padding and stay zero.
        The parameters themselves must already hold the checkpointed weights."""
        lo, hi = self.begin, self.begin + self.count
        self.m.zero_()
        self.v.zero_()
        self.refresh_master()
        for sh in shards:
            a, b = max(lo, sh["begin"]), min(hi, sh["begin"] + sh["count"])
            if a >= b:
                continue
            src, dst = slice(a - sh["begin"], b - sh["begin"]), slice(a - lo, b - lo)
            self.m[dst].copy_(sh["m"][src])
            self.v[dst].copy_(sh["v"][src])
            if self.master is not None and sh.get("master") is not None:
                self.master[dst].copy_(sh["master"][src])
        if shards and shards[0].get("scaler"):
            self.scaler.load_state_dict(shards[0]["scaler"])

    def _fold_autograd_grads(self):
        for p in self.fp.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def step(self):
        self._fold_autograd_grads()
        P = self.ranks
        s = self.scaler
        if self.cuda:
            a = DpAdamArgs()
            self.epoch += 1
            a.rank, a.ranks, a.epoch, a.grid_ctas = self.rank, P, self.epoch, self.grid
            for r in range(P):
                a.grad_ptrs[r] = self.sym.ptrs[r] + self._g_off
                a.signal_ptrs[r] = self.sym.ptrs[r] + self._s_off
                if self.low:
                    a.param_lp_ptrs[r] = self.sym.ptrs[r] + self._p_off
                else:
                    a.param_fp_ptrs[r] = self.sym.ptrs[r] + self._p_off
            a.master = _lib.ptr(self.master)
            a.m, a.v, a.gsum = self.m.data_ptr(), self.v.data_ptr(), self.gsum.data_ptr()
            a.begin, a.count = self.begin, self.count
            a.lr, a.beta1, a.beta2, a.eps = self.lr, self.beta1, self.beta2, self.eps
            a.weight_decay, a.max_grad_norm = self.weight_decay, self.max_grad_norm
            on = s.enabled
            a.growth, a.backoff = (s.growth, s.backoff) if on else (1.0, 1.0)
            a.min_scale, a.max_scale = (s.min_scale, s.max_scale) if on else (1.0, 1.0)
            a.window = s.window
            a.scaler = s.state.data_ptr()
            a.block_part, a.grid_bar = self.block_part.data_ptr(), self.grid_bar.data_ptr()
            a.grid_bar_base = (2 * self.grid * self.calls) & 0xFFFFFFFF
            self.calls += 1
            a.grad_mul = 1.0 / P if self.average else 1.0
            _lib.check(_lib.lib().cgk_dp_adam_step(ctypes.byref(a), _lib.stream_ptr()), "cgk_dp_adam_step")
            _lib.count_launch()
            if a.grid_bar_base > 2 ** 31:
                torch.cuda.current_stream().synchronize()
                self.grid_bar.zero_()
                self.calls = 0
            return
        # ---- CPU ranks: all-reduce + the same update rule on the owned slice + all-gather ----
        if P > 1:
            dist.all_reduce(self.grad, group=self.group)
            if self.average:
                self.grad.mul_(1.0 / P)
        g = self.grad
        found = not bool(torch.isfinite(g).all())
        inv = 1.0 / s._host["scale"] if s.enabled else 1.0
        if s.host_update(found):
            return
        g = g * inv
        if self.max_grad_norm > 0:
            norm = float(g.norm())
            if norm > self.max_grad_norm:
                g = g * (self.max_grad_norm / (norm + 1e-6))
        sl = slice(self.begin, self.begin + self.count)
        gs = g[sl]
        t = s._host["step"]
        p = self.master if self.master is not None else self.fp.flat[sl]
        if self.weight_decay > 0:
            p.mul_(1.0 - self.lr * self.weight_decay)
        self.m.mul_(self.beta1).add_(gs, alpha=1 - self.beta1)
        self.v.mul_(self.beta2).addcmul_(gs, gs, value=1 - self.beta2)
        p.sub_(self.lr * (self.m / (1 - self.beta1 ** t)) / (torch.sqrt(self.v / (1 - self.beta2 ** t)) + self.eps))
        new_slice = p.to(self.fp.flat.dtype)
        if P > 1:
            parts = [torch.empty_like(new_slice) for _ in range(P)]
            dist.all_gather(parts, new_slice.contiguous(), group=self.group)
            self.fp.flat.copy_(torch.cat(parts))
        elif self.master is not None:
            self.fp.flat[sl].copy_(new_slice)


class DataParallel:
    """Glue for ``Trainer``: with ``DPFusedAdam`` the gradient reduction happens inside the
    optimizer step, so ``reduce_gradients`` has nothing to do; it exists so that a plain
    ``FusedAdam`` can be used with NCCL all-reduce as the comparison point."""

    def __init__(self, model, rank, world, dev, group=None):
        self.model, self.rank, self.world = model, rank, world
        self.group = group if group is not None else (dist.group.WORLD if world > 1 else None)

    def make_optimizer(self, **kw):
        return DPFusedAdam(self.model.parameters(), self.group, **kw)

    def reduce_gradients(self, opt):
        if isinstance(opt, DPFusedAdam) or self.world == 1:
            return
        dist.all_reduce(opt.grad, group=self.group)
        opt.grad.mul_(1.0 / self.world)
