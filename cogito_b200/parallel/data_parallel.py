"""Data parallelism whose optimizer step is fused with its collectives: gradient all-reduce
over NVLink peer memory + loss-scale unscale / overflow check + global-norm clip + Adam +
broadcast of the new weights (csrc/comm/dp_adam.cu).  The reduce-scatter runs bucket by
bucket on a side stream while the backward pass is still producing gradients
(``cgk_dp_bucket_reduce``); one kernel after the last bucket takes the skip / clip decision,
updates and broadcasts (``cgk_dp_adam_finish``).

Each rank keeps the fp32 master weights and Adam moments of its part of every bucket only
(sharded optimizer state); parameters and gradients live in symmetric memory so that peers
can read gradients and write updated weights.

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


class DpBucketArgs(Structure):
    _fields_ = [("rank", c_int32), ("ranks", c_int32), ("epoch", c_int32), ("bucket", c_int32), ("grid_ctas", c_int32),
                ("grad_ptrs", c_void_p * 8), ("signal_ptrs", c_void_p * 8), ("gsum", c_void_p),
                ("begin", c_int64), ("count", c_int64), ("block_part", c_void_p), ("arrive", c_void_p),
                ("stats", c_void_p)]


class DpFinishArgs(Structure):
    _fields_ = [("rank", c_int32), ("ranks", c_int32), ("epoch", c_int32), ("nbuckets", c_int32), ("grid_ctas", c_int32),
                ("param_lp_ptrs", c_void_p * 8), ("param_fp_ptrs", c_void_p * 8), ("signal_ptrs", c_void_p * 8),
                ("master", c_void_p), ("m", c_void_p), ("v", c_void_p), ("gsum", c_void_p),
                ("n", c_int64), ("bucket_len", c_int64),
                ("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float),
                ("weight_decay", c_float), ("max_grad_norm", c_float), ("grad_mul", c_float),
                ("growth", c_float), ("backoff", c_float), ("min_scale", c_float), ("max_scale", c_float),
                ("window", c_int32), ("scaler", c_void_p), ("bucket_stats", c_void_p), ("ext_stats", c_void_p),
                ("arrive", c_void_p)]


MAX_BUCKETS = 64        # CGK_DP_MAX_BUCKETS


class DPFusedAdam:
    """Adam over a data-parallel group.  Same surface as ``FusedAdam`` (``fp``, ``grad``,
    ``scaler``, ``zero_grad``, ``step``); gradients are summed over the group inside ``step``
    (use ``average=True`` to divide by the group size).

    The flat parameter vector is cut into buckets of ``bucket_elems`` elements; in every bucket
    rank r owns the r-th of P equal parts (``segments``).  After :meth:`arm` (the trainer calls
    it before the last backward pass of a step) the hooks installed by :meth:`attach_overlap`
    start the reduce-scatter of a bucket on a side stream as soon as the backward pass has gone
    past it; :meth:`step` reduces whatever is left and runs the update kernel."""

    def __init__(self, params, group=None, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 scaler: GradScaler | None = None, max_grad_norm: float = 0.0, average: bool = True,
                 bucket_elems: int = 16 * 1024 * 1024, reduce_ctas: int = 24):
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
        unit = 8 * P
        n = (n_guess + unit - 1) // unit * unit
        self.n = n
        L = max(unit, (int(bucket_elems) + unit - 1) // unit * unit)
        if (n + L - 1) // L > MAX_BUCKETS:
            L = ((n + MAX_BUCKETS - 1) // MAX_BUCKETS + unit - 1) // unit * unit
        self.bucket_len = L
        self.nbuckets = (n + L - 1) // L
        # (flat begin, count, offset in the local state vectors) of the part of every bucket this rank owns
        self.segments = []
        off = 0
        for b in range(self.nbuckets):
            len_b = min(L, n - b * L)
            self.segments.append((b * L + self.rank * (len_b // P), len_b // P, off))
            off += len_b // P
        self.low = params[0].dtype != torch.float32
        if self.cuda:
            Lk = _lib.lib()
            Lk.cgk_dp_bucket_reduce.argtypes = [POINTER(DpBucketArgs), c_void_p]
            Lk.cgk_dp_adam_finish.argtypes = [POINTER(DpFinishArgs), c_void_p]
            p_bytes = (n * esize + 255) // 256 * 256
            g_bytes = (n * 4 + 255) // 256 * 256
            s_bytes = (Lk.cgk_dp_signal_bytes(P) + 255) // 256 * 256
            self.sym = SymmetricBuffer(p_bytes + g_bytes + s_bytes, dev, group)
            self._p_off, self._g_off, self._s_off = 0, p_bytes, p_bytes + g_bytes
            alloc = lambda ne, dt: self.sym.view(0, (ne,), dt)
            self.fp = FlatParams(params, alloc=alloc, pad_to=unit)
            assert self.fp.total == n
            self.grad = self.sym.view(self._g_off, (n,), torch.float32)
        else:
            self.fp = FlatParams(params, pad_to=unit)
            self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        for p, g in zip(self.fp.params, self.fp.views(self.grad)):
            p.main_grad = g
        per = n // P
        self.count = per
        self.master = self._gather_owned(self.fp.flat).float().clone() if self.low else None
        self.m = torch.zeros(per, dtype=torch.float32, device=dev)
        self.v = torch.zeros(per, dtype=torch.float32, device=dev)
        self.epoch = 0
        self._armed = False
        self._launched = set()
        self.ext_stats_fn = None      # callable(local {norm^2, overflow} tensor) -> tensor agreed by a larger group
        if self.cuda:
            self.reduce_ctas = max(1, min(int(reduce_ctas), 1024))
            # buckets that are still open when the backward pass ends (the tied embedding's) are reduced
            # with the whole GPU: nothing else runs then, and a CTA pulls only ~7 GB/s from its peers
            self.tail_ctas = max(self.reduce_ctas, min(1024, torch.cuda.get_device_properties(dev).multi_processor_count))
            self.gsum = torch.empty(per, dtype=torch.float32, device=dev)
            self.block_part = torch.zeros(self.nbuckets, 2 * self.tail_ctas, dtype=torch.float32, device=dev)
            self.arrive = torch.zeros(self.nbuckets + 1, dtype=torch.int32, device=dev)
            self.bucket_stats = torch.zeros(self.nbuckets, 2, dtype=torch.float32, device=dev)
            self.comm_stream = torch.cuda.Stream(device=dev)

    # -- ownership -------------------------------------------------------------------------
    def _gather_owned(self, flat: torch.Tensor) -> torch.Tensor:
        """The owned parts of a flat vector, bucket after bucket."""
        return torch.cat([flat[b:b + c] for b, c, _ in self.segments])

    def _scatter_owned(self, flat: torch.Tensor, owned: torch.Tensor) -> None:
        for b, c, o in self.segments:
            flat[b:b + c].copy_(owned[o:o + c])

    # -- overlap with the backward pass ----------------------------------------------------
    def arm(self) -> None:
        """The next backward pass is the last one of this step: buckets may leave as they fill."""
        self._armed = True
        self._launched = set()

    def attach_overlap(self, model) -> int:
        """Installs hooks on the sub-modules of ``model`` (the members of its ModuleLists, else its
        children): when the gradient of a sub-module's input arrives, every parameter from that
        sub-module to the end of the flat vector has its gradient, and the buckets that lie wholly
        in that range are reduced on the side stream.  This relies on the usual layout: sub-modules
        are registered in the order in which the forward pass uses them, and a parameter shared
        between an early and a late use is registered with the early one (tied embeddings are).
        ``COGITO_DP_OVERLAP=0`` leaves the hooks out.  Returns the number of hooks."""
        import os
        if os.environ.get("COGITO_DP_OVERLAP", "1") in ("", "0"):
            return 0
        first = {}
        for p, o in zip(self.fp.params, self.fp.offsets):
            first[id(p)] = o
        mods = []
        for child in model.children():
            mods.extend(list(child) if isinstance(child, torch.nn.ModuleList) else [child])
        count = 0
        for mod in mods:
            offs = [first[id(p)] for p in mod.parameters() if id(p) in first]
            if not offs:
                continue
            lo = min(offs)
            # every parameter registered after this module must also sit behind it in the flat vector
            def pre_hook(module, args, lo=lo):
                x = args[0] if args else None
                if torch.is_tensor(x) and x.requires_grad and torch.is_grad_enabled():
                    x.register_hook(lambda g, lo=lo: self.gradients_ready_from(lo))
            mod.register_forward_pre_hook(pre_hook)
            count += 1
        return count

    def gradients_ready_from(self, offset: int) -> None:
        """All gradients at flat positions >= offset are complete (in stream order)."""
        if not (self._armed and self.cuda and self.ranks > 1):
            return
        todo = [b for b in range(self.nbuckets) if b * self.bucket_len >= offset and b not in self._launched]
        if not todo:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.comm_stream.wait_event(ev)
        for b in sorted(todo, reverse=True):
            self._reduce_bucket(b, self.comm_stream)

    def _reduce_bucket(self, b: int, stream, ctas: int | None = None) -> None:
        P = self.ranks
        begin, count, off = self.segments[b]
        a = DpBucketArgs()
        a.rank, a.ranks, a.epoch, a.bucket, a.grid_ctas = self.rank, P, self.epoch + 1, b, ctas or self.reduce_ctas
        for r in range(P):
            a.grad_ptrs[r] = self.sym.ptrs[r] + self._g_off
            a.signal_ptrs[r] = self.sym.ptrs[r] + self._s_off
        a.gsum = self.gsum.data_ptr() + 4 * off
        a.begin, a.count = begin, count
        a.block_part = self.block_part[b].data_ptr()
        a.arrive = self.arrive[b:b + 1].data_ptr()
        a.stats = self.bucket_stats[b].data_ptr()
        _lib.check(_lib.lib().cgk_dp_bucket_reduce(ctypes.byref(a), stream.cuda_stream), "cgk_dp_bucket_reduce")
        _lib.count_launch()
        self._launched.add(b)

    @property
    def params(self):
        return self.fp.params

    def zero_grad(self):
        self.grad.zero_()
        for p in self.fp.params:
            p.grad = None

    def refresh_master(self):
        """Re-read this rank's fp32 master weights from the parameters (after a weight load)."""
        if self.master is not None:
            self.master.copy_(self._gather_owned(self.fp.flat).float())

    def check(self) -> None:
        """Reads the device status word (synchronises).  A wait on a peer that ran out makes the
        kernels return early; the counters they use are reset here and the failure is raised."""
        if not self.cuda:
            return
        code, where, block, aux = _lib.read_status()
        if code != 0:
            self.arrive.zero_()
            self._launched = set()
            self._armed = False
            from ..utils.failure import RankFailure
            raise RankFailure(f"data-parallel step gave up waiting for a peer: code={code} where={where} block={block} aux={aux}")

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
        d.update(segments=[list(sg) for sg in self.segments], n=self.n, ranks=self.ranks, scaler=self.scaler.state_dict())
        return d

    def load_resharded(self, shards) -> None:
        """Restore from the shards of a run with ANY data-parallel size (a rank was lost, or ranks
        were added).  Parameters start at the same offsets of the flat vector whatever the group
        size (only the padding at its end depends on it), so this rank's slice is filled from the
        overlap of each of its parts with the parts of each old shard; positions no old shard covers
        are padding and stay zero.
        The parameters themselves must already hold the checkpointed weights."""
        self.m.zero_()
        self.v.zero_()
        self.refresh_master()
        for sh in shards:
            old = sh.get("segments") or [(sh["begin"], sh["count"], 0)]     # shards written before bucketing: one part
            for ob, oc, oo in old:
                for nb_, nc, no in self.segments:
                    a, b = max(nb_, ob), min(nb_ + nc, ob + oc)
                    if a >= b:
                        continue
                    src, dst = slice(oo + a - ob, oo + b - ob), slice(no + a - nb_, no + b - nb_)
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
            Lk = _lib.lib()
            main = torch.cuda.current_stream()
            rest = [b for b in range(self.nbuckets) if b not in self._launched] if self._armed else list(range(self.nbuckets))
            if not self._armed:
                self._launched = set()
            for b in sorted(rest, reverse=True):       # what the backward pass did not release: on the main stream
                self._reduce_bucket(b, main, self.tail_ctas)
            if len(rest) < self.nbuckets:
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                main.wait_event(ev)
            self._armed = False
            self._launched = set()
            self.epoch += 1
            ext = None
            if self.ext_stats_fn is not None:
                ext = self.ext_stats_fn(self.bucket_stats.sum(0))
            a = DpFinishArgs()
            a.rank, a.ranks, a.epoch, a.nbuckets, a.grid_ctas = self.rank, P, self.epoch, self.nbuckets, 0
            for r in range(P):
                a.signal_ptrs[r] = self.sym.ptrs[r] + self._s_off
                if self.low:
                    a.param_lp_ptrs[r] = self.sym.ptrs[r] + self._p_off
                else:
                    a.param_fp_ptrs[r] = self.sym.ptrs[r] + self._p_off
            a.master = _lib.ptr(self.master)
            a.m, a.v, a.gsum = self.m.data_ptr(), self.v.data_ptr(), self.gsum.data_ptr()
            a.n, a.bucket_len = self.n, self.bucket_len
            a.lr, a.beta1, a.beta2, a.eps = self.lr, self.beta1, self.beta2, self.eps
            a.weight_decay, a.max_grad_norm = self.weight_decay, self.max_grad_norm
            on = s.enabled
            a.growth, a.backoff = (s.growth, s.backoff) if on else (1.0, 1.0)
            a.min_scale, a.max_scale = (s.min_scale, s.max_scale) if on else (1.0, 1.0)
            a.window = s.window
            a.scaler = s.state.data_ptr()
            a.bucket_stats = self.bucket_stats.data_ptr()
            a.ext_stats = _lib.ptr(ext)
            a.arrive = self.arrive[self.nbuckets:].data_ptr()
            a.grad_mul = 1.0 / P if self.average else 1.0
            _lib.check(Lk.cgk_dp_adam_finish(ctypes.byref(a), _lib.stream_ptr()), "cgk_dp_adam_finish")
            _lib.count_launch()
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
        gs = self._gather_owned(g)
        t = s._host["step"]
        owned = self.master if self.master is not None else self._gather_owned(self.fp.flat)
        if self.weight_decay > 0:
            owned.mul_(1.0 - self.lr * self.weight_decay)
        self.m.mul_(self.beta1).add_(gs, alpha=1 - self.beta1)
        self.v.mul_(self.beta2).addcmul_(gs, gs, value=1 - self.beta2)
        owned.sub_(self.lr * (self.m / (1 - self.beta1 ** t)) / (torch.sqrt(self.v / (1 - self.beta2 ** t)) + self.eps))
        new_owned = owned.to(self.fp.flat.dtype)
        if P > 1:
            parts = [torch.empty_like(new_owned) for _ in range(P)]
            dist.all_gather(parts, new_owned.contiguous(), group=self.group)
            L = self.bucket_len
            for r, part in enumerate(parts):            # rank r's parts, bucket after bucket
                o = 0
                for b in range(self.nbuckets):
                    c = min(L, self.n - b * L) // P
                    self.fp.flat[b * L + r * c:b * L + (r + 1) * c].copy_(part[o:o + c])
                    o += c
        else:
            self._scatter_owned(self.fp.flat, new_owned)


class DataParallel:
    """Glue for ``Trainer``: with ``DPFusedAdam`` the gradient reduction happens inside the
    optimizer step, so ``reduce_gradients`` has nothing to do; it exists so that a plain
    ``FusedAdam`` can be used with NCCL all-reduce as the comparison point."""

    def __init__(self, model, rank, world, dev, group=None):
        self.model, self.rank, self.world = model, rank, world
        self.group = group if group is not None else (dist.group.WORLD if world > 1 else None)

    def make_optimizer(self, **kw):
        opt = DPFusedAdam(self.model.parameters(), self.group, **kw)
        opt.attach_overlap(self.model)
        return opt

    def reduce_gradients(self, opt):
        if isinstance(opt, DPFusedAdam) or self.world == 1:
            return
        dist.all_reduce(opt.grad, group=self.group)
        opt.grad.mul_(1.0 / self.world)
