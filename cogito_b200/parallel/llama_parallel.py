"""Llama under DP x TP x PP: tensor-parallel blocks (grouped-query attention with RoPE,
SwiGLU) on the fused all-gather->GEMM / GEMM->reduce-scatter kernels, split into pipeline
stages that run the 1F1B schedule, replicated over data-parallel groups whose optimizer step
is the fused all-reduce + Adam kernel.

Reference counterparts: cg_3d_parallel / cg_pipeline_parallel / cg_tensor_parallel_linear
(include/cg_pipeline.h:44-75,170-200), rank mapping src/pipeline/pipeline.c (tp fastest, then
pp, then dp); the transformer switches of cg_transformer_config (include/cg_transformer.h).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from ..models.llama import LlamaConfig
from ..nn.modules import RMSNorm
from ..nn.transformer import packed_attention
from ..ops import loss as L
from ..ops import misc as M
from ..optim.fused import FusedAdam, GradScaler
from ..utils import rng
from .data_parallel import DPFusedAdam
from .groups import ParallelContext
from .interleaved import InterleavedExecutor
from .pipeline import PipelineExecutor
from .tensor_parallel import _ColumnRow, _LMHead, _VocabParallelCE
from .tp_ops import TPWorkspace
from ..utils.recompute import checkpoint


class TPLlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, ws: TPWorkspace, device=None, dtype=None):
        super().__init__()
        P = ws.ranks
        if cfg.n_head % P or cfg.n_kv_head % P or cfg.d_ff % P:
            raise ValueError("heads, kv heads and d_ff must divide evenly over the tensor-parallel ranks")
        self.cfg, self.ws = cfg, ws
        self.hq, self.hk, self.hd, self.fl = cfg.n_head // P, cfg.n_kv_head // P, cfg.head_dim, cfg.d_ff // P
        d = cfg.d_model
        mk = lambda *shape: nn.Parameter(rng.normal_(torch.empty(*shape, device=device, dtype=dtype), cfg.init_std,
                                                      rng.layer_generator(ws.rank + 1)))
        self.norm1 = RMSNorm(d, cfg.norm_eps, device=device, dtype=dtype)
        self.norm2 = RMSNorm(d, cfg.norm_eps, device=device, dtype=dtype)
        self.w_qkv = mk((self.hq + 2 * self.hk) * self.hd, d)        # local q heads | k heads | v heads
        self.w_proj = mk(d, self.hq * self.hd)
        self.w_gate_up = mk(2 * self.fl, d)                          # local gate | up
        self.w_down = mk(d, self.fl)
        for p in list(self.norm1.parameters()) + list(self.norm2.parameters()):
            p.tp_replicated = True
        self._rope = None

    def _tables(self, device):
        if self._rope is None or self._rope[0].device != device:
            self._rope = M.rope_tables(self.cfg.max_seq_len, self.hd, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, x_shard, batch_tokens):
        B, T = batch_tokens
        Hq, Hk, D = self.hq, self.hk, self.hd
        rope = self._tables(x_shard.device)

        # on GPUs the QKV GEMM rotates the q and k heads in its epilogue; elsewhere attention does it
        fused_rope = x_shard.is_cuda and D in (64, 128) and ((Hq + 2 * Hk) * D) % 32 == 0

        def attend(qkv):
            x = qkv.view(B, T, Hq + 2 * Hk, D)
            o = packed_attention(x, Hq, Hk, causal=True, scale=1.0 / math.sqrt(D), rope=None if fused_rope else rope)
            return o.reshape(B * T, Hq * D)

        h, xr = self.norm1(x_shard, passthrough=True)     # gradients of the stream meet inside the norm's backward
        x_shard = _ColumnRow.apply(h, self.w_qkv, None, self.w_proj, None, None, xr, self.ws, attend,
                                   (rope[0], rope[1], (Hq + Hk) * D, D, T) if fused_rope else None)
        h, xr = self.norm2(x_shard, passthrough=True)
        return _ColumnRow.apply(h, self.w_gate_up, None, self.w_down, None, None, xr, self.ws, M.swiglu)


class _SeqShardEmbedding(torch.autograd.Function):
    """Vocabulary-sharded embedding whose output is the sequence-sharded residual stream:
    x_shard = reduce_scatter_r(wte_r[ids])."""

    @staticmethod
    def forward(ctx, ids, wte, ws):
        B, T = ids.shape
        P, r = ws.ranks, ws.rank
        partial = M.embedding(ids, wte.detach(), None, r * wte.shape[0]).reshape(B * T, -1)
        if P > 1:
            shard = torch.empty(B * T // P, partial.shape[1], device=partial.device, dtype=partial.dtype)
            dist.reduce_scatter_tensor(shard, partial.contiguous(), group=ws.group)
        else:
            shard = partial
        ctx.save_for_backward(ids)
        ctx.ws, ctx.wte = ws, wte
        return shard

    @staticmethod
    def backward(ctx, dshard):
        (ids,) = ctx.saved_tensors
        ws, wte = ctx.ws, ctx.wte
        P, r = ws.ranks, ws.rank
        B, T = ids.shape
        dshard = dshard.contiguous()
        if P > 1:
            full = torch.empty(B * T, dshard.shape[1], device=dshard.device, dtype=dshard.dtype)
            dist.all_gather_into_tensor(full, dshard, group=ws.group)
        else:
            full = dshard
        Vl = wte.shape[0]
        local = ids.reshape(-1) - r * Vl
        ok = (local >= 0) & (local < Vl)
        target = wte.main_grad if getattr(wte, "main_grad", None) is not None else torch.zeros_like(wte, dtype=torch.float32)
        target.index_add_(0, local[ok], full[ok].float())
        return None, (None if getattr(wte, "main_grad", None) is not None else target.to(wte.dtype)), None


class LlamaStage(nn.Module):
    """The layers [first, last) of a Llama on one pipeline stage, tensor-parallel over `ws`.
    The first stage owns the embedding, the last the final norm, the output head and the loss."""

    def __init__(self, cfg: LlamaConfig, ws: TPWorkspace, stage: int, num_stages: int, device=None, dtype=None):
        super().__init__()
        if cfg.n_layer % num_stages:
            raise ValueError("layers must divide evenly over the pipeline stages")
        self.cfg, self.ws, self.stage, self.S = cfg, ws, stage, num_stages
        self.recompute = False         # True: per-block activation recomputation
        per = cfg.n_layer // num_stages
        self.first, self.last = stage * per, (stage + 1) * per
        P = ws.ranks
        if cfg.vocab_size % P:
            raise ValueError("vocabulary must divide evenly over the tensor-parallel ranks")
        Vl = cfg.vocab_size // P
        mk = lambda *shape: nn.Parameter(rng.normal_(torch.empty(*shape, device=device, dtype=dtype), cfg.init_std,
                                                      rng.layer_generator(ws.rank + 1)))
        self.wte = mk(Vl, cfg.d_model) if stage == 0 else None
        self.blocks = nn.ModuleList([TPLlamaBlock(cfg, ws, device, dtype) for _ in range(per)])
        if stage == num_stages - 1:
            self.norm_f = RMSNorm(cfg.d_model, cfg.norm_eps, device=device, dtype=dtype)
            for p in self.norm_f.parameters():
                p.tp_replicated = True
            self.w_head = mk(Vl, cfg.d_model)
        else:
            self.norm_f, self.w_head = None, None

    def forward(self, x, batch_tokens, targets=None, grad_scale=1.0):
        """x: token ids [B, T] on the first stage, else the sequence-sharded activation
        [B*T/tp, d].  Returns the activation, or the loss on the last stage when targets are given."""
        if self.stage == 0:
            x = _SeqShardEmbedding.apply(x, self.wte, self.ws)
        for blk in self.blocks:
            x = checkpoint(blk, x, batch_tokens) if self.recompute else blk(x, batch_tokens)
        if self.stage != self.S - 1:
            return x
        logits = _LMHead.apply(self.norm_f(x), self.w_head, self.ws)
        if targets is None:
            return logits
        return _VocabParallelCE.apply(logits, targets, grad_scale, self.ws)

    def ordered_parameters(self):
        rep = [p for p in self.parameters() if getattr(p, "tp_replicated", False)]
        shd = [p for p in self.parameters() if not getattr(p, "tp_replicated", False)]
        return rep + shd


def shard_llama_state(full, stage: LlamaStage) -> None:
    """Copy the weights of a single-device ``Llama`` into this rank's stage / TP shards."""
    cfg, ws = stage.cfg, stage.ws
    P, r = ws.ranks, ws.rank
    Hq, Hk, D, d, I = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_model, cfg.d_ff
    hq, hk, fl, Vl = Hq // P, Hk // P, I // P, cfg.vocab_size // P

    def put(dst, src):
        with torch.no_grad():
            dst.copy_(src.to(dst.device, dst.dtype))

    if stage.wte is not None:
        put(stage.wte, full.wte[r * Vl:(r + 1) * Vl])
    for fb, tb in zip(list(full.blocks)[stage.first:stage.last], stage.blocks):
        put(tb.norm1.weight, fb.norm1.weight); put(tb.norm2.weight, fb.norm2.weight)
        w = fb.attn.qkv.weight
        q, k, v = w[:Hq * D].view(Hq, D, d), w[Hq * D:(Hq + Hk) * D].view(Hk, D, d), w[(Hq + Hk) * D:].view(Hk, D, d)
        put(tb.w_qkv, torch.cat([q[r * hq:(r + 1) * hq].reshape(-1, d), k[r * hk:(r + 1) * hk].reshape(-1, d),
                                 v[r * hk:(r + 1) * hk].reshape(-1, d)]))
        put(tb.w_proj, fb.attn.proj.weight[:, r * hq * D:(r + 1) * hq * D])
        gu = fb.mlp.gate_up.weight
        put(tb.w_gate_up, torch.cat([gu[r * fl:(r + 1) * fl], gu[I + r * fl:I + (r + 1) * fl]]))
        put(tb.w_down, fb.mlp.down.weight[:, r * fl:(r + 1) * fl])
    if stage.norm_f is not None:
        put(stage.norm_f.weight, full.norm_f.weight)
        put(stage.w_head, full.lm_head.weight[r * Vl:(r + 1) * Vl])


class ModelParallelStats:
    """(overflow flag, sum of squares of the gradients) of one rank -> of the whole model replica, i.e.
    over the tensor- and pipeline-parallel ranks of one data-parallel replica.  Parameters that every
    tensor-parallel rank holds in full (the first ``n_rep`` elements of the flat gradient, identical on
    those ranks once their gradients have been all-reduced) are counted once."""

    def __init__(self, ctx, opt, n_rep: int):
        self.ctx, self.opt, self.n_rep = ctx, opt, n_rep

    def __call__(self, found: torch.Tensor, norm_sq: torch.Tensor) -> None:
        c = self.ctx.coords
        if c.tp > 1 and self.n_rep and c.tp_rank != 0:
            g = torch.nan_to_num(self.opt.grad[:self.n_rep], nan=0.0, posinf=0.0, neginf=0.0)
            norm_sq -= (g * g).sum()
        dist.all_reduce(found, op=dist.ReduceOp.MAX, group=self.ctx.mp_group)
        dist.all_reduce(norm_sq, op=dist.ReduceOp.SUM, group=self.ctx.mp_group)


class ReplicaStatsDP:
    """The same for the fused data-parallel optimizer: its bucket kernels leave (sum of squares,
    overflow) of the parts of the DATA-PARALLEL-SUMMED gradient that this rank owns; the sum over
    every rank of the job (data-, tensor- and pipeline-parallel) is what the whole model sees.
    Replicated parameters (flat positions below ``n_rep``) are counted on tensor-parallel rank 0 only."""

    def __init__(self, ctx, opt, n_rep: int):
        self.ctx, self.opt, self.n_rep = ctx, opt, n_rep

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        st = local.clone()
        c = self.ctx.coords
        if c.tp > 1 and self.n_rep and c.tp_rank != 0:
            for b, cnt, off in self.opt.segments:
                hi = min(b + cnt, self.n_rep)
                if hi > b:
                    g = torch.nan_to_num(self.opt.gsum[off:off + hi - b], nan=0.0, posinf=0.0, neginf=0.0)
                    st[0] -= (g * g).sum()
        dist.all_reduce(st)
        return st.contiguous()


class Trainer3D:
    """One rank of a DP x TP x PP job.  ``step(ids, targets)`` takes this data-parallel replica's
    batch [M * micro_batch, T] (every rank of the replica passes the same tensors) and runs M
    micro-batches through the 1F1B schedule, then the optimizer step: replicated-parameter
    gradients are summed over the TP group, all gradients averaged over the DP group inside
    the fused Adam kernel (or a plain all-reduce on CPU ranks)."""

    def __init__(self, cfg: LlamaConfig, ctx: ParallelContext, device, num_microbatches: int, micro_batch: int, seq_len: int,
                 lr: float = 1e-4, loss_scale: float | None = 65536.0, max_grad_norm: float = 1.0, weight_decay: float = 0.0,
                 virtual_stages: int = 1, recompute: str | None = None, comm_sms: int = 8):
        """virtual_stages > 1: every pipeline rank holds that many model chunks (virtual stage = chunk * pp +
        pp_rank) and the step runs the interleaved 1F1B schedule (parallel/interleaved.py); the number of
        micro-batches must then be a multiple of pp.
        recompute: None keeps every activation; "block" drops the activations inside each transformer
        block and recomputes them in backward (``utils.recompute.checkpoint``); "stage" keeps only each
        in-flight micro-batch's stage input and runs the stage's forward pass a second time (1F1B
        executor only).  comm_sms: SMs that persistent GEMM kernels leave free for the pipeline's
        transfer kernels, which run on a side stream beside them."""
        if recompute not in (None, "block", "stage"):
            raise ValueError("recompute must be None, 'block' or 'stage'")
        self.cfg, self.ctx, self.device = cfg, ctx, torch.device(device)
        self.M, self.mb, self.T = num_microbatches, micro_batch, seq_len
        cuda = self.device.type == "cuda"
        dtype = torch.bfloat16 if cuda else None
        c = ctx.coords
        tokens = micro_batch * seq_len
        if tokens % c.tp:
            raise ValueError("micro_batch * seq_len must divide by the tensor-parallel size")
        max_ctas = 0
        if cuda and c.pp > 1 and comm_sms > 0:
            from ..ops.gemm import set_default_max_ctas
            max_ctas = max(8, torch.cuda.get_device_properties(self.device).multi_processor_count - comm_sms)
            set_default_max_ctas(max_ctas)
        self.ws = TPWorkspace(self.device, ctx.tp_group if c.tp > 1 else None, max_rows=tokens,
                              max_cols=max(cfg.d_model, 1), max_ctas=max_ctas)
        V = self.V = virtual_stages
        self.stages = [LlamaStage(cfg, self.ws, ch * c.pp + c.pp_rank, c.pp * V, self.device, dtype) for ch in range(V)]
        for st in self.stages:
            st.recompute = recompute == "block"
        self.stage = self.stages[0]
        self.scaler = GradScaler(self.device, enabled=loss_scale is not None, init_scale=loss_scale or 1.0)
        # replicated parameters of every chunk first: their gradients are one contiguous slice
        allp = [p for st in self.stages for p in st.parameters()]
        params = [p for p in allp if getattr(p, "tp_replicated", False)] + [p for p in allp if not getattr(p, "tp_replicated", False)]
        kw = dict(lr=lr, scaler=self.scaler, max_grad_norm=max_grad_norm, weight_decay=weight_decay)
        # Loss scaling and norm clipping decide per step from statistics of the WHOLE replica (all tp x pp
        # ranks): an overflow seen on one pipeline stage must skip the step on every stage.  The fused
        # data-parallel optimizer computes its statistics over the data-parallel ranks of one (tp, pp)
        # coordinate; with model parallelism on top they are summed over all ranks of the job between
        # its reduce kernels and its update kernel (ReplicaStatsDP), on the GPU, and the update kernel
        # takes the agreed pair instead of its own exchange.  CPU ranks (gloo) average the gradients with
        # one all-reduce and step FusedAdam with the replica-wide statistics.
        need_replica_stats = c.tp * c.pp > 1 and (loss_scale is not None or max_grad_norm > 0)
        fused_dp = c.dp > 1 and (cuda or not need_replica_stats)
        self._dp_allreduce = c.dp > 1 and not fused_dp
        self.opt = DPFusedAdam(params, ctx.dp_group, **kw) if fused_dp else FusedAdam(params, **kw)
        self.n_rep = 0
        for p, o in zip(self.opt.fp.params, self.opt.fp.offsets):
            if getattr(p, "tp_replicated", False):
                self.n_rep = o + (p.numel() + 7) // 8 * 8
        if c.tp * c.pp > 1 and isinstance(self.opt, FusedAdam):
            self.opt.stats_sync = ModelParallelStats(ctx, self.opt, self.n_rep)
        if need_replica_stats and isinstance(self.opt, DPFusedAdam):
            self.opt.ext_stats_fn = ReplicaStatsDP(ctx, self.opt, self.n_rep)
        act_dtype = torch.bfloat16 if cuda else torch.float32
        if V == 1:
            self.pipe = PipelineExecutor(c.pp_rank, c.pp, num_microbatches, ctx.prev_stage, ctx.next_stage,
                                         (tokens // c.tp, cfg.d_model), act_dtype, self.device,
                                         links=ctx.pipeline_links, recompute=recompute == "stage")
        else:
            self.pipe = InterleavedExecutor(c.pp_rank, ctx.pp_ranks if c.pp > 1 else [0], V, num_microbatches,
                                            (tokens // c.tp, cfg.d_model), act_dtype, self.device)

    def load_from(self, full) -> None:
        """Take this rank's stage / tensor-parallel shards from a single-device ``Llama``."""
        for st in self.stages:
            shard_llama_state(full, st)
        self.opt.refresh_master()

    def step(self, ids: torch.Tensor, targets: torch.Tensor):
        M_, mb, T = self.M, self.mb, self.T
        self.opt.zero_grad()
        ids_m, tgt_m = ids.view(M_, mb, T), targets.view(M_, mb, T)
        scale = self.scaler.scale_tensor if (self.scaler.enabled and self.device.type == "cuda") else self.scaler.scale

        c = self.ctx.coords
        last_virtual = c.pp * self.V - 1

        def chunk_fn(ch):
            stage, is_last = self.stages[ch], ch * c.pp + c.pp_rank == last_virtual

            def stage_fn(x, m):
                return stage(x, (mb, T), tgt_m[m] if is_last else None, scale / M_)
            return stage_fn

        first = [ids_m[m] for m in range(M_)]
        loss = self.pipe.run(chunk_fn(0), first_inputs=first) if self.V == 1 else self.pipe.run([chunk_fn(ch) for ch in range(self.V)], first)
        if self.ctx.coords.tp > 1 and self.n_rep:
            dist.all_reduce(self.opt.grad[:self.n_rep], group=self.ctx.tp_group)
        if self._dp_allreduce:
            dist.all_reduce(self.opt.grad, group=self.ctx.dp_group)
            self.opt.grad.mul_(1.0 / self.ctx.coords.dp)
        self.opt.step()           # overflow flag and gradient norm are those of the whole replica (stats_sync)
        return loss
