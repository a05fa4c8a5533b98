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
    """Same model and step with PyTorch library kernels; data parallel (DDP) for N > 1."""

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


def build_job(args, rank, world, dev):
    if args.impl == "torch":
        return TorchJob(args, rank, world, dev)
    return CogitoJob(args, rank, world, dev)
