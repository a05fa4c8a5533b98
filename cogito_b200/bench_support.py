"""Job construction for bench.py: the framework's own GPT-2 training job and the
PyTorch-library baseline of the identical configuration."""
from __future__ import annotations

import math

import torch
from torch import nn


class _Job:
    vocab = 50304
    flops_per_token = 0.0

    def step(self, ids, targets):
        raise NotImplementedError

    def launch_count(self) -> int:
        return 0

    def reset_launch_count(self) -> None:
        pass


class CogitoJob(_Job):
    """GPT-2 through the framework's public API (models.GPT2 + FusedAdam + Trainer)."""

    def __init__(self, args, rank, world, dev):
        from .models.gpt2 import GPT2, GPT2Config
        from .optim.fused import FusedAdam, GradScaler
        from .ops import _lib
        from .train import Trainer

        self._lib = _lib
        torch.manual_seed(0)
        cfg = GPT2Config(n_layer=args.layers, max_seq_len=args.seq_len)
        self.vocab = cfg.vocab_size
        if world > 1 and args.parallelism == "tp":
            from .parallel.tensor_parallel import build_tp_gpt2
            self.model, parallel = build_tp_gpt2(cfg, rank, world, dev, micro_tokens=args.micro_batch * args.seq_len)
        else:
            self.model = GPT2(cfg, device=dev, dtype=torch.bfloat16)
            parallel = None
            if world > 1:
                from .parallel.data_parallel import DataParallel
                parallel = DataParallel(self.model, rank, world, dev)
        scaler = GradScaler(dev, enabled=False)
        params = getattr(self.model, "_ordered", None) or list(self.model.parameters())
        if world > 1 and args.parallelism == "dp":
            self.opt = parallel.make_optimizer(lr=1e-4, scaler=scaler)      # fused all-reduce + Adam kernel
        else:
            self.opt = FusedAdam(params, lr=1e-4, scaler=scaler)
        if parallel is not None and hasattr(parallel, "attach"):
            parallel.attach(self.opt)
        mb = args.micro_batch
        self.dp = world if (world > 1 and args.parallelism == "dp") else 1
        self.rank = rank
        self.trainer = Trainer(self.model, self.opt, micro_batch=mb, parallel=parallel)
        self.flops_per_token = _gpt2_flops_per_token(cfg, args.seq_len)

    def step(self, ids, targets):
        if self.dp > 1:
            per = ids.shape[0] // self.dp
            ids = ids[self.rank * per:(self.rank + 1) * per]
            targets = targets[self.rank * per:(self.rank + 1) * per]
        return self.trainer.step(ids, targets)

    def launch_count(self):
        return self._lib.launches()

    def reset_launch_count(self):
        self._lib.reset_launches()


def _gpt2_flops_per_token(cfg, seq_len):
    per_layer = 2 * (4 * cfg.d_model * cfg.d_model + 2 * cfg.d_model * cfg.d_ff)
    attn = 2 * 2 * seq_len * cfg.d_model / 2
    head = 2 * cfg.d_model * cfg.vocab_size
    return 3.0 * (cfg.n_layer * (per_layer + attn) + head)


# ---------------------------------------------------------------------------
# PyTorch-library baseline (cuBLAS GEMMs, SDPA attention, fused AdamW, NCCL)
# ---------------------------------------------------------------------------
class _TorchBlock(nn.Module):
    def __init__(self, d, h, ff):
        super().__init__()
        self.h = h
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.up, self.down = nn.Linear(d, ff), nn.Linear(ff, d)

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        a = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, C))
        return x + self.down(nn.functional.gelu(self.up(self.ln2(x)), approximate="tanh"))


class _TorchGPT2(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.wte = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq_len, cfg.d_model)
        self.blocks = nn.ModuleList([_TorchBlock(cfg.d_model, cfg.n_head, cfg.d_ff) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, cfg.init_std)

    def forward(self, ids, targets):
        T = ids.shape[1]
        x = self.wte(ids) + self.wpe(torch.arange(T, device=ids.device))[None]
        for b in self.blocks:
            x = b(x)
        logits = nn.functional.linear(self.ln_f(x), self.wte.weight)
        return nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))


class TorchJob(_Job):
    """Same model and step with PyTorch library kernels (fp32 parameters under bf16 autocast); data
    parallel (DDP) for N > 1.  The comparison point of the data-parallel measurement."""

    def __init__(self, args, rank, world, dev):
        from .models.gpt2 import GPT2Config
        torch.manual_seed(0)
        cfg = GPT2Config(n_layer=args.layers, max_seq_len=args.seq_len)
        self.vocab = cfg.vocab_size
        self.model = _TorchGPT2(cfg).to(dev)
        self.world, self.rank, self.mb = world, rank, args.micro_batch
        self.ddp = None
        if world > 1:
            self.ddp = nn.parallel.DistributedDataParallel(self.model, device_ids=[dev.index])
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=1e-4, weight_decay=0.0, fused=True)
        self.flops_per_token = _gpt2_flops_per_token(cfg, args.seq_len)
        self.dev = dev

    def step(self, ids, targets):
        ids = ids.to(self.dev, non_blocking=True)
        targets = targets.to(self.dev, non_blocking=True)
        if self.world > 1:
            per = ids.shape[0] // self.world
            ids, targets = ids[self.rank * per:(self.rank + 1) * per], targets[self.rank * per:(self.rank + 1) * per]
        B = ids.shape[0]
        n_micro = max(1, math.ceil(B / self.mb))
        self.opt.zero_grad(set_to_none=True)
        total = 0.0
        m = self.ddp if self.ddp is not None else self.model
        for i in range(n_micro):
            sl = slice(i * self.mb, min(B, (i + 1) * self.mb))
            sync = (i == n_micro - 1) or self.ddp is None
            ctx = torch.autocast("cuda", dtype=torch.bfloat16)
            if self.ddp is not None and not sync:
                with self.ddp.no_sync(), ctx:
                    loss = m(ids[sl], targets[sl]) / n_micro
                    loss.backward()
            else:
                with ctx:
                    loss = m(ids[sl], targets[sl]) / n_micro
                loss.backward()
            total = total + loss.detach()
        self.opt.step()
        return total


# ---------------------------------------------------------------------------
# PyTorch-library baseline of the tensor-parallel configuration: the unfused design
# (NCCL all-gather, cuBLAS GEMM, cuBLAS GEMM, NCCL reduce-scatter) of
# cg_tp_column_parallel_forward / cg_tp_row_parallel_forward
# (src/pipeline/tensor_parallel.c:31-105) with sequence-sharded activations, SDPA attention
# and fused AdamW.  Same sharding as the framework's own model, none of its kernels.
# ---------------------------------------------------------------------------
class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = torch.distributed.get_world_size(group)
        out = torch.empty(x.shape[0] * P, *x.shape[1:], device=x.device, dtype=x.dtype)
        torch.distributed.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        P = torch.distributed.get_world_size(ctx.group)
        out = torch.empty(g.shape[0] // P, *g.shape[1:], device=g.device, dtype=g.dtype)
        torch.distributed.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = torch.distributed.get_world_size(group)
        out = torch.empty(x.shape[0] // P, *x.shape[1:], device=x.device, dtype=x.dtype)
        torch.distributed.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        P = torch.distributed.get_world_size(ctx.group)
        out = torch.empty(g.shape[0] * P, *g.shape[1:], device=g.device, dtype=g.dtype)
        torch.distributed.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _AllReduceSum(torch.autograd.Function):
    """Forward all-reduce, identity backward (the summed quantity feeds every rank's loss alike)."""

    @staticmethod
    def forward(ctx, x, group, op):
        x = x.clone()
        torch.distributed.all_reduce(x, op=op, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class _TorchTPBlock(nn.Module):
    def __init__(self, d, heads_local, hd, ff_local, group):
        super().__init__()
        self.group, self.hl, self.hd = group, heads_local, hd
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * heads_local * hd)
        self.proj = nn.Linear(heads_local * hd, d, bias=False)
        self.proj_bias = nn.Parameter(torch.zeros(d))
        self.up = nn.Linear(d, ff_local)
        self.down = nn.Linear(ff_local, d, bias=False)
        self.down_bias = nn.Parameter(torch.zeros(d))

    def _gather(self, x):
        return _AllGatherRows.apply(x, self.group) if self.group is not None else x

    def _scatter(self, x):
        return _ReduceScatterRows.apply(x, self.group) if self.group is not None else x

    def forward(self, x, B, T):
        h = self._gather(self.ln1(x))                                   # [B*T, d]
        q, k, v = self.qkv(h).view(B, T, 3, self.hl, self.hd).permute(2, 0, 3, 1, 4)
        a = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        a = a.transpose(1, 2).reshape(B * T, self.hl * self.hd)
        x = x + self._scatter(self.proj(a)) + self.proj_bias
        h = self._gather(self.ln2(x))
        h = nn.functional.gelu(self.up(h), approximate="tanh")
        return x + self._scatter(self.down(h)) + self.down_bias


class _TorchTPGPT2(nn.Module):
    def __init__(self, cfg, rank, world, group):
        super().__init__()
        from .parallel.tensor_parallel import head_span
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        hd = cfg.d_model // cfg.n_head
        _, hl = head_span(cfg.n_head, world, rank)
        self.vl = cfg.vocab_size // world
        self.wte = nn.Parameter(torch.empty(self.vl, cfg.d_model).normal_(0.0, cfg.init_std))
        self.wpe = nn.Parameter(torch.empty(cfg.max_seq_len, cfg.d_model).normal_(0.0, cfg.init_std))
        self.blocks = nn.ModuleList([_TorchTPBlock(cfg.d_model, hl, hd, cfg.d_ff // world, group) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0.0, cfg.init_std)

    def forward(self, ids, targets):
        B, T = ids.shape
        P, r, g = self.world, self.rank, self.group
        loc = ids.reshape(-1) - r * self.vl
        ok = (loc >= 0) & (loc < self.vl)
        emb = self.wte[loc.clamp(0, self.vl - 1)] * ok[:, None].to(self.wte.dtype)          # [B*T, d] partial
        rows = B * T // P
        x = _ReduceScatterRows.apply(emb, g) if g is not None else emb
        pos = (torch.arange(rows, device=ids.device) + r * rows) % T
        x = x + self.wpe[pos]
        for blk in self.blocks:
            x = blk(x, B, T)
        h = self.ln_f(x)
        h = _AllGatherRows.apply(h, g) if g is not None else h
        logits = nn.functional.linear(h, self.wte).float()                                # [B*T, V/P]
        tg = targets.reshape(-1) - r * self.vl
        mine = (tg >= 0) & (tg < self.vl)
        mx = logits.max(-1).values.detach()
        if g is not None:
            mx = _AllReduceSum.apply(mx, g, torch.distributed.ReduceOp.MAX)
        se = torch.exp(logits - mx[:, None]).sum(-1)
        tl = logits.gather(1, tg.clamp(0, self.vl - 1)[:, None]).squeeze(1) * mine.to(logits.dtype)
        if g is not None:
            se = _AllReduceSum.apply(se, g, torch.distributed.ReduceOp.SUM)
            tl = _AllReduceSum.apply(tl, g, torch.distributed.ReduceOp.SUM)
        return (mx + torch.log(se) - tl).mean()


class TorchTPJob(_Job):
    """The named configuration (tensor parallel over all ranks) on PyTorch library kernels: bf16
    parameters and activations, NCCL collectives, cuBLAS, SDPA, fused AdamW."""

    def __init__(self, args, rank, world, dev):
        from .models.gpt2 import GPT2Config
        torch.manual_seed(rank)
        cfg = GPT2Config(n_layer=args.layers, max_seq_len=args.seq_len)
        self.vocab = cfg.vocab_size
        group = torch.distributed.group.WORLD if world > 1 else None
        self.model = _TorchTPGPT2(cfg, rank, world, group).to(dev, torch.bfloat16)
        self.replicated = [p for n, p in self.model.named_parameters()
                           if n == "wpe" or ".ln" in n or n.startswith("ln_f") or n.endswith("proj_bias") or n.endswith("down_bias")]
        self.world, self.group, self.mb, self.dev = world, group, args.micro_batch, dev
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=1e-4, weight_decay=0.0, fused=True)
        self.flops_per_token = _gpt2_flops_per_token(cfg, args.seq_len)

    def step(self, ids, targets):
        ids = ids.to(self.dev, non_blocking=True)
        targets = targets.to(self.dev, non_blocking=True)
        B = ids.shape[0]
        n_micro = max(1, math.ceil(B / self.mb))
        self.opt.zero_grad(set_to_none=True)
        total = 0.0
        for i in range(n_micro):
            sl = slice(i * self.mb, min(B, (i + 1) * self.mb))
            loss = self.model(ids[sl], targets[sl]) / n_micro
            loss.backward()
            total = total + loss.detach()
        if self.world > 1:
            # parameters every rank holds in full saw only this rank's rows
            flat = torch.cat([p.grad.reshape(-1) for p in self.replicated])
            torch.distributed.all_reduce(flat, group=self.group)
            o = 0
            for p in self.replicated:
                p.grad.copy_(flat[o:o + p.numel()].view_as(p.grad))
                o += p.numel()
        self.opt.step()
        return total


def build_job(args, rank, world, dev):
    if args.impl == "torch":
        if args.parallelism == "tp":
            return TorchTPJob(args, rank, world, dev)
        return TorchJob(args, rank, world, dev)
    return CogitoJob(args, rank, world, dev)
