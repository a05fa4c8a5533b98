"""Tensor parallelism with sequence-sharded activations (Megatron-style) built on the
fused kernels: every column-parallel GEMM is an all-gather -> GEMM kernel, every
row-parallel GEMM a GEMM -> reduce-scatter kernel, and their backward passes are the
duals (dX of a column layer is GEMM -> reduce-scatter, dX of a row layer is
all-gather -> GEMM; the dW GEMMs reuse the gathered buffer the forward produced).

Between blocks the residual stream, LayerNorm and dropout see ``[tokens / TP, d]``.
Parameters that every rank holds in full (norm weights, row-parallel biases, position
embeddings) get partial gradients per rank; they are flagged ``tp_replicated`` and
all-reduced over the TP group before the optimizer step.

Reference counterparts: cg_tensor_parallel_linear, cg_tp_column_parallel_forward and
cg_tp_row_parallel_forward (include/cg_pipeline.h:170-175,
src/pipeline/tensor_parallel.c:31-105), which have no backward and gather the column
shards along the wrong dimension.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from ..nn.modules import LayerNorm
from ..nn.transformer import packed_attention
from ..ops import _lib
from ..ops import functional as F
from ..ops import misc as M
from ..ops.gemm import gemm
from ..utils import rng
from .tp_ops import TPWorkspace, ag_gemm, gemm_rs


def _wgrad(dy2, x2, w):
    return F._weight_grad(dy2, x2, w)


def _bgrad(dy2, b):
    return F._bias_grad(dy2, b)


class _ColumnRow(torch.autograd.Function):
    """y_shard = residual + act(AG(x_shard) W1^T + b1) W2^T + b2 with W1 column-sharded and
    W2 row-sharded: the tensor-parallel MLP, and (with `inner`) the attention block."""

    @staticmethod
    def forward(ctx, x_shard, w1, b1, w2, b2, act, residual, ws, inner, rope=None):
        """rope: (cos, sin, cols, head_dim, T) applies the rotary embedding to the first ``cols`` columns
        of the first GEMM's output in its epilogue (the q and k heads of a QKV projection); ``inner``
        then sees rotated heads, and the backward pass undoes the rotation on the gradient."""
        z = None
        if act not in (None, "none"):
            z = torch.empty(x_shard.shape[0] * ws.ranks, w1.shape[0], device=x_shard.device, dtype=x_shard.dtype)
        spec = None if rope is None else (rope[0], rope[1], rope[2], rope[3], rope[4], 0, False)
        h, gathered = ag_gemm(ws, x_shard, w1, bias=b1, act=act, aux_out=z, rope=spec)
        ctx.rope = rope
        ctx.slot = _lib.grad_slot()
        if inner is not None:
            # differentiable function applied between the two GEMMs (attention); it runs
            # under its own small autograd graph, replayed in backward
            with torch.enable_grad():
                h_in = h.detach().requires_grad_(True)
                h_out = inner(h_in)
            ctx.inner_io = (h_in, h_out)
            h2 = h_out.detach()
        else:
            ctx.inner_io = None
            h2 = h
        y = gemm_rs(ws, h2, w2, bias=b2, residual=residual)
        ctx.save_for_backward(gathered, w1, w2, z if z is not None else torch.empty(0), h2)
        ctx.act, ctx.b1, ctx.b2, ctx.ws = act, b1, b2, ws
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        prev = _lib.set_grad_slot(ctx.slot)
        try:
            return _ColumnRow._backward(ctx, dy)
        finally:
            _lib.set_grad_slot(prev)

    @staticmethod
    def _backward(ctx, dy):
        gathered, w1, w2, z, h2 = ctx.saved_tensors
        ws, act = ctx.ws, ctx.act
        dy = dy.contiguous()
        has_act = act not in (None, "none")
        if has_act and ctx.inner_io is None:
            dz, dy_g = _ag_gemm_bwd(ws, dy, w2, aux_in=z, dact=act)       # (AG(dy) W2) * act'(z)
        else:
            dz, dy_g = _ag_gemm_bwd(ws, dy, w2)
        dw2 = _wgrad(dy_g, h2, w2)
        db2 = _bgrad(dy, ctx.b2)
        if ctx.inner_io is not None:
            h_in, h_out = ctx.inner_io
            (dz,) = torch.autograd.grad(h_out, h_in, dz)
            dz = dz.contiguous()
            if ctx.rope is not None:
                cos, sin, cols, D, T = ctx.rope
                M.rope_apply_(dz.view(-1, T, dz.shape[1] // D, D)[:, :, :cols // D], cos, sin, backward=True)
            if has_act:
                dz = F.unary_backward(act, z, dz)
        dw1 = _wgrad(dz, gathered, w1)
        db1 = _bgrad(dz, ctx.b1)
        dx = gemm_rs(ws, dz, w1, b_mn=True)
        return dx, dw1, db1, dw2, db2, None, (dy if ctx.has_res else None), None, None, None


def _ag_gemm_bwd(ws, dy_shard, w, aux_in=None, dact=None):
    """(AG(dy_shard) @ W) [* act'(aux_in)] for a row-sharded W [N, K_local]; returns (dx, gathered dy).
    The activation derivative is applied in the GEMM's epilogue."""
    return ag_gemm(ws, dy_shard, w, b_mn=True, aux_in=aux_in, dact=dact, keep=False)


def head_span(n_head: int, ranks: int, rank: int):
    """(first head, number of heads) of `rank`: the first ``n_head % ranks`` ranks hold one more."""
    base, extra = divmod(n_head, ranks)
    return rank * base + min(rank, extra), base + (1 if rank < extra else 0)


class TPAttention(nn.Module):
    def __init__(self, d_model, n_head, ws: TPWorkspace, causal=True, init_std=0.02, device=None, dtype=None):
        super().__init__()
        if n_head < ws.ranks:
            raise ValueError("tensor parallelism needs at least one attention head per rank")
        # heads that do not divide evenly (GPT-2-small: 12 heads over 8 ranks) are dealt out
        # 2,2,2,2,1,1,1,1: only the attention core is unbalanced, every GEMM keeps its fused path
        first, count = head_span(n_head, ws.ranks, ws.rank)
        self.ws, self.h_local, self.hd, self.causal = ws, count, d_model // n_head, causal
        nl = 3 * self.h_local * self.hd
        g = rng.layer_generator(ws.rank + 1)
        self.w_qkv = nn.Parameter(rng.normal_(torch.empty(nl, d_model, device=device, dtype=dtype), init_std, g))
        self.b_qkv = nn.Parameter(torch.zeros(nl, device=device, dtype=dtype))
        self.w_proj = nn.Parameter(rng.normal_(torch.empty(d_model, self.h_local * self.hd, device=device, dtype=dtype),
                                               init_std, rng.layer_generator(ws.rank + 1)))
        self.b_proj = nn.Parameter(torch.zeros(d_model, device=device, dtype=dtype))
        self.b_proj.tp_replicated = True
        self.seq_len = None

    def forward(self, h_shard, residual, batch_tokens, ws=None):
        B, T = batch_tokens
        Hl, D = self.h_local, self.hd

        def attend(qkv):
            x = qkv.view(B, T, 3 * Hl, D)
            o = packed_attention(x, Hl, Hl, causal=self.causal, scale=1.0 / math.sqrt(D))
            return o.reshape(B * T, Hl * D)

        return _ColumnRow.apply(h_shard, self.w_qkv, self.b_qkv, self.w_proj, self.b_proj, None, residual,
                                ws or self.ws, attend)


class TPMLP(nn.Module):
    def __init__(self, d_model, d_ff, ws: TPWorkspace, act="gelu", init_std=0.02, device=None, dtype=None):
        super().__init__()
        P = ws.ranks
        if d_ff % P:
            raise ValueError("d_ff must divide evenly over the tensor-parallel ranks")
        self.ws, self.act = ws, act
        fl = d_ff // P
        self.w1 = nn.Parameter(rng.normal_(torch.empty(fl, d_model, device=device, dtype=dtype), init_std,
                                           rng.layer_generator(ws.rank + 1)))
        self.b1 = nn.Parameter(torch.zeros(fl, device=device, dtype=dtype))
        self.w2 = nn.Parameter(rng.normal_(torch.empty(d_model, fl, device=device, dtype=dtype), init_std,
                                           rng.layer_generator(ws.rank + 1)))
        self.b2 = nn.Parameter(torch.zeros(d_model, device=device, dtype=dtype))
        self.b2.tp_replicated = True

    def forward(self, h_shard, residual, ws=None):
        return _ColumnRow.apply(h_shard, self.w1, self.b1, self.w2, self.b2, self.act, residual, ws or self.ws, None)


class TPBlock(nn.Module):
    def __init__(self, d_model, n_head, d_ff, ws, eps=1e-5, init_std=0.02, device=None, dtype=None):
        super().__init__()
        self.ln1 = LayerNorm(d_model, eps, device=device, dtype=dtype)
        self.attn = TPAttention(d_model, n_head, ws, True, init_std, device, dtype)
        self.ln2 = LayerNorm(d_model, eps, device=device, dtype=dtype)
        self.mlp = TPMLP(d_model, d_ff, ws, "gelu", init_std, device, dtype)
        for p in list(self.ln1.parameters()) + list(self.ln2.parameters()):
            p.tp_replicated = True

    def forward(self, x_shard, batch_tokens, ws=None):
        h, xr = self.ln1(x_shard, passthrough=True)       # gradients of the stream meet inside the norm's backward
        x_shard = self.attn(h, xr, batch_tokens, ws)
        h, xr = self.ln2(x_shard, passthrough=True)
        return self.mlp(h, xr, ws)


class _VocabParallelEmbedding(torch.autograd.Function):
    """x_shard = reduce_scatter_r(wte_r[ids]) + wpe[pos]; vocabulary rows are sharded."""

    @staticmethod
    def forward(ctx, ids, wte, wpe, ws):
        B, T = ids.shape
        P, r = ws.ranks, ws.rank
        Vl = wte.shape[0]
        partial = M.embedding(ids, wte.detach(), None, r * Vl).reshape(B * T, -1)
        rows = B * T // P
        if P > 1:
            shard = torch.empty(rows, partial.shape[1], device=partial.device, dtype=partial.dtype)
            dist.reduce_scatter_tensor(shard, partial.contiguous(), group=ws.group)
        else:
            shard = partial
        pos = (torch.arange(rows, device=ids.device) + r * rows) % T
        shard = (shard.float() + wpe.detach()[pos].float()).to(partial.dtype)
        ctx.save_for_backward(ids, pos)
        ctx.ws, ctx.params = ws, (wte, wpe)
        ctx.slot = _lib.grad_slot()
        return shard

    @staticmethod
    def backward(ctx, dshard):
        ids, pos = ctx.saved_tensors
        ws = ctx.ws
        wte, wpe = ctx.params
        P, r = ws.ranks, ws.rank
        B, T = ids.shape
        dshard = dshard.contiguous()
        if P > 1:
            full = torch.empty(B * T, dshard.shape[1], device=dshard.device, dtype=dshard.dtype)
            dist.all_gather_into_tensor(full, dshard, group=ws.group)
        else:
            full = dshard
        prev = _lib.set_grad_slot(ctx.slot)
        g_wte, g_wpe = _lib.main_grad_of(wte), _lib.main_grad_of(wpe)
        _lib.set_grad_slot(prev)
        own = g_wte is None
        if own:
            g_wte = torch.zeros(wte.shape, device=wte.device, dtype=torch.float32)
        Vl = wte.shape[0]
        if wte.is_cuda:
            _lib.check(_lib.lib().cgk_embedding_backward(
                ids.contiguous().data_ptr(), full.data_ptr(), g_wte.data_ptr(), None, B * T, full.shape[1], T,
                r * Vl, Vl, _lib.stream_ptr()), "cgk_embedding_backward")
            _lib.count_launch()
        else:
            local = (ids.reshape(-1) - r * Vl)
            ok = (local >= 0) & (local < Vl)
            g_wte.index_add_(0, local[ok], full.float()[ok])
        own_p = g_wpe is None
        if own_p:
            g_wpe = torch.zeros(wpe.shape, device=wpe.device, dtype=torch.float32)
        g_wpe.index_add_(0, pos, dshard.float())
        return None, (g_wte.to(wte.dtype) if own else None), (g_wpe.to(wpe.dtype) if own_p else None), None


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy over vocabulary-sharded logits [R, V/P]; d(logits) overwrites the logits."""

    @staticmethod
    def forward(ctx, logits, targets, grad_scale, ws):
        R, Vl = logits.shape
        P, r = ws.ranks, ws.rank
        tg = targets.reshape(-1).contiguous()
        if logits.is_cuda:
            L = _lib.lib()
            mx, sm, tl = (torch.empty(R, device=logits.device, dtype=torch.float32) for _ in range(3))
            _lib.check(L.cgk_ce_stats(logits.data_ptr(), tg.data_ptr(), r * Vl, mx.data_ptr(), sm.data_ptr(),
                                      tl.data_ptr(), R, Vl, logits.stride(0), _lib.stream_ptr()), "cgk_ce_stats")
            _lib.count_launch()
        else:
            lf = logits.float()
            mx = lf.max(-1).values
            sm = torch.exp(lf - mx[:, None]).sum(-1)
            loc = tg - r * Vl
            ok = (loc >= 0) & (loc < Vl)
            tl = torch.where(ok, lf.gather(1, loc.clamp(0, Vl - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
        gmax = mx.clone()
        if P > 1:
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=ws.group)
        st = torch.stack([sm * torch.exp(mx - gmax), tl])
        if P > 1:
            dist.all_reduce(st, group=ws.group)
        lse = gmax + torch.log(st[0])
        loss = (lse - st[1]).mean()
        scale = grad_scale if isinstance(grad_scale, torch.Tensor) else None
        scale_f = (1.0 if scale is not None else float(grad_scale)) / R
        if logits.is_cuda:
            sp = scale.reshape(1).float().contiguous() if scale is not None else None
            _lib.check(_lib.lib().cgk_ce_backward(logits.data_ptr(), tg.data_ptr(), r * Vl, lse.contiguous().data_ptr(),
                                                  logits.data_ptr(), R, Vl, logits.stride(0), scale_f,
                                                  _lib.ptr(sp), -100, _lib.stream_ptr()), "cgk_ce_backward")
            _lib.count_launch()
            d = logits
        else:
            p = torch.exp(logits.float() - lse[:, None])
            loc = tg - r * Vl
            ok = (loc >= 0) & (loc < Vl)
            p[torch.arange(R)[ok], loc[ok]] -= 1.0
            d = (p * scale_f * (float(scale) if scale is not None else 1.0)).to(logits.dtype)
        ctx.save_for_backward(d)
        return loss

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d, None, None, None


class _LMHead(torch.autograd.Function):
    """logits_local = AG(h_shard) wte_r^T; backward: dh_shard = RS(dlogits wte_r), dwte_r += dlogits^T AG(h)."""

    @staticmethod
    def forward(ctx, h_shard, wte, ws):
        logits, gathered = ag_gemm(ws, h_shard, wte)
        ctx.save_for_backward(gathered, wte)
        ctx.ws = ws
        ctx.slot = _lib.grad_slot()
        return logits

    @staticmethod
    def backward(ctx, dlogits):
        gathered, wte = ctx.saved_tensors
        prev = _lib.set_grad_slot(ctx.slot)
        try:
            dw = _wgrad(dlogits, gathered, wte)
        finally:
            _lib.set_grad_slot(prev)
        dh = gemm_rs(ctx.ws, dlogits, wte, b_mn=True)
        return dh, dw, None


class TPGPT2(nn.Module):
    """GPT-2 with every matmul tensor-parallel: vocabulary-sharded embedding / output head,
    head-sharded attention, column/row-sharded MLP, sequence-sharded residual stream."""

    def __init__(self, cfg, ws: TPWorkspace, device=None, dtype=None, ws2: TPWorkspace | None = None):
        super().__init__()
        self.cfg, self.ws = cfg, ws
        # a second workspace turns on the two-halves-on-two-streams forward / backward pass
        self.workspaces = [ws] + ([ws2] if ws2 is not None else [])
        self._streams = [torch.cuda.Stream(device=ws.device), torch.cuda.Stream(device=ws.device)] if ws2 is not None else []
        P = ws.ranks
        if cfg.vocab_size % P:
            raise ValueError("vocabulary must divide evenly over the tensor-parallel ranks")
        Vl = cfg.vocab_size // P
        self.wte = nn.Parameter(rng.normal_(torch.empty(Vl, cfg.d_model, device=device, dtype=dtype), cfg.init_std,
                                            rng.layer_generator(ws.rank + 1)))
        self.wpe = nn.Parameter(rng.normal_(torch.empty(cfg.max_seq_len, cfg.d_model, device=device, dtype=dtype),
                                            cfg.init_std, rng.layer_generator()))
        self.wpe.tp_replicated = True
        self.blocks = nn.ModuleList([TPBlock(cfg.d_model, cfg.n_head, cfg.d_ff, ws, cfg.norm_eps, cfg.init_std,
                                             device, dtype) for _ in range(cfg.n_layer)])
        self.ln_f = LayerNorm(cfg.d_model, cfg.norm_eps, device=device, dtype=dtype)
        for p in self.ln_f.parameters():
            p.tp_replicated = True

    def _forward_part(self, ids, targets, grad_scale, ws):
        B, T = ids.shape
        ws.begin_step()              # the gathered activations of the previous pass are dead
        x = _VocabParallelEmbedding.apply(ids, self.wte, self.wpe, ws)
        for blk in self.blocks:
            x = blk(x, (B, T), ws)
        h = self.ln_f(x)
        logits = _LMHead.apply(h, self.wte, ws)
        if targets is None:
            return logits
        return _VocabParallelCE.apply(logits, targets, grad_scale, ws)

    def forward(self, ids, targets=None, grad_scale=1.0):
        """With a second workspace (``overlap=True`` at construction) and targets, the batch is cut in
        two halves that run on two streams at once: while the all-gather / reduce-scatter kernels of
        one half wait for NVLink, the attention and weight-gradient kernels of the other half have
        the SMs (the fused kernels are capped to a part of the GPU for that).  Each half accumulates
        its parameter gradients into its own buffer (gradient slots); ``TPGradSync`` adds them up."""
        B, T = ids.shape
        if len(self.workspaces) < 2 or targets is None or not ids.is_cuda or B < 2 or (B // 2) * T % (128 * self.ws.ranks):
            return self._forward_part(ids, targets, grad_scale, self.ws)
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        half = B // 2
        parts = [(ids[:half], targets[:half]), (ids[half:], targets[half:])]
        # each half's loss is a mean over its own rows: scale its gradient by its share of the batch
        share = [half / B, (B - half) / B]
        xs = [None, None]

        def on(i, fn):
            """Issue fn on half i's stream with half i's gradient slot selected."""
            prev = _lib.set_grad_slot(i)
            try:
                with torch.cuda.stream(self._streams[i]):
                    return fn()
            finally:
                _lib.set_grad_slot(prev)

        # The halves are issued layer by layer in turn, so that both streams always have work queued
        # and the backward pass (which autograd issues in the reverse of this order) alternates too.
        for i in (0, 1):
            self._streams[i].wait_event(start)
            self.workspaces[i].begin_step()
            xs[i] = on(i, lambda i=i: _VocabParallelEmbedding.apply(parts[i][0], self.wte, self.wpe, self.workspaces[i]))
        for blk in self.blocks:
            for i in (0, 1):
                xs[i] = on(i, lambda i=i: blk(xs[i], (parts[i][0].shape[0], T), self.workspaces[i]))
        losses = []
        for i in (0, 1):
            def tail(i=i):
                logits = _LMHead.apply(self.ln_f(xs[i]), self.wte, self.workspaces[i])
                return _VocabParallelCE.apply(logits, parts[i][1], grad_scale * share[i], self.workspaces[i])
            losses.append(on(i, tail))
        for st in self._streams:
            main.wait_stream(st)
        return losses[0] * share[0] + losses[1] * share[1]

    def ordered_parameters(self):
        """Replicated parameters first, so their gradients are one contiguous slice."""
        rep = [p for p in self.parameters() if getattr(p, "tp_replicated", False)]
        shd = [p for p in self.parameters() if not getattr(p, "tp_replicated", False)]
        return rep, shd


class TPGradSync:
    """All-reduces the gradients of the replicated parameters over the TP group; with the two-stream
    forward pass it first gives every parameter a second gradient buffer (one per half of the
    batch) and adds the two up before the optimizer step."""

    def __init__(self, model: TPGPT2):
        self.model = model
        self.n_rep = None
        self.group = model.ws.group
        self.ranks = model.ws.ranks
        self.grad2 = None

    def attach(self, opt):
        rep, _ = self.model.ordered_parameters()
        n = 0
        for p, o in zip(opt.fp.params, opt.fp.offsets):
            if getattr(p, "tp_replicated", False):
                n = o + (p.numel() + 7) // 8 * 8
        self.n_rep = n
        if len(self.model.workspaces) > 1:
            self.grad2 = torch.zeros_like(opt.grad)
            for p, a, b in zip(opt.fp.params, opt.fp.views(opt.grad), opt.fp.views(self.grad2)):
                p.main_grad_slots = [a, b]

    def reduce_gradients(self, opt):
        if self.grad2 is not None:
            opt.grad.add_(self.grad2)
            self.grad2.zero_()
        if self.ranks > 1 and self.n_rep:
            dist.all_reduce(opt.grad[:self.n_rep], group=self.group)


def build_tp_gpt2(cfg, rank, world, dev, group=None, micro_tokens=16384, overlap: bool | None = None,
                  fused_ctas: int = 56):
    """overlap: run the two halves of every batch on two streams at once (see ``TPGPT2.forward``).
    None = on for GPU groups of four or more ranks, where the collectives dominate the step;
    ``COGITO_TP_OVERLAP=0`` / ``=1`` force it off / on.  fused_ctas: CTAs of each fused collective kernel in that mode (the two
    halves' kernels must fit on the GPU together, with room left for the compute kernels)."""
    import os
    if group is None and world > 1:
        group = dist.group.WORLD
    cuda = torch.device(dev).type == "cuda"
    if overlap is None:
        env = os.environ.get("COGITO_TP_OVERLAP", "")
        overlap = cuda and (env not in ("", "0") if env != "" else world >= 4)
    overlap = bool(overlap) and cuda and world > 1 and micro_tokens % (2 * 128 * world) == 0
    tokens = micro_tokens // 2 if overlap else micro_tokens
    # room for the gathered input of every column-parallel GEMM of one pass (two per block and
    # the output head), which the backward pass reads again
    arena = (2 * cfg.n_layer + 1) * ((tokens * cfg.d_model * 2 + 255) // 256 * 256)
    mk = lambda: TPWorkspace(dev, group, max_rows=tokens, max_cols=cfg.d_model, arena_bytes=arena,
                             max_ctas=fused_ctas if overlap else 0)
    ws = mk()
    ws2 = mk() if overlap else None
    model = TPGPT2(cfg, ws, device=dev, dtype=torch.bfloat16 if cuda else None, ws2=ws2)
    rep, shd = model.ordered_parameters()
    model._ordered = rep + shd
    return model, TPGradSync(model)


def shard_gpt2_state(full, tp: TPGPT2) -> None:
    """Copy the weights of a single-device GPT2 (`full`) into this rank's shards of `tp`."""
    P, r = tp.ws.ranks, tp.ws.rank
    cfg = tp.cfg
    H, D = cfg.n_head, cfg.d_model // cfg.n_head
    h0, Hl = head_span(H, P, r)

    def put(dst, src):
        with torch.no_grad():
            dst.copy_(src.to(dst.device, dst.dtype))

    Vl = cfg.vocab_size // P
    put(tp.wte, full.wte[r * Vl:(r + 1) * Vl])
    put(tp.wpe, full.wpe)
    for fb, tb in zip(full.blocks, tp.blocks):
        put(tb.ln1.weight, fb.norm1.weight); put(tb.ln1.bias, fb.norm1.bias)
        put(tb.ln2.weight, fb.norm2.weight); put(tb.ln2.bias, fb.norm2.bias)
        wq = fb.attn.qkv.weight.view(3, H, D, cfg.d_model)[:, h0:h0 + Hl]
        bq = fb.attn.qkv.bias.view(3, H, D)[:, h0:h0 + Hl]
        put(tb.attn.w_qkv, wq.reshape(3 * Hl * D, cfg.d_model))
        put(tb.attn.b_qkv, bq.reshape(3 * Hl * D))
        put(tb.attn.w_proj, fb.attn.proj.weight[:, h0 * D:(h0 + Hl) * D])
        put(tb.attn.b_proj, fb.attn.proj.bias)
        fl = cfg.d_ff // P
        put(tb.mlp.w1, fb.mlp.up.weight[r * fl:(r + 1) * fl]); put(tb.mlp.b1, fb.mlp.up.bias[r * fl:(r + 1) * fl])
        put(tb.mlp.w2, fb.mlp.down.weight[:, r * fl:(r + 1) * fl]); put(tb.mlp.b2, fb.mlp.down.bias)
    put(tp.ln_f.weight, full.ln_f.weight); put(tp.ln_f.bias, full.ln_f.bias)
