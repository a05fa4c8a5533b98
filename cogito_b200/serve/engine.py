"""INT4 Llama serving engine and the draft/verify speculative decoding loop.

One engine step runs ``Tq`` new tokens per sequence through the model against the paged INT4
KV cache: RMSNorm -> INT4 GEMM (q|k|v) -> RoPE at the sequence's own positions -> quantise and
append K/V -> attention over the cache -> INT4 GEMM (+ residual) -> RMSNorm -> INT4 GEMM
(gate|up) -> SwiGLU -> INT4 GEMM (+ residual).  The cache lengths move only when the caller
commits, so a verify pass over ``gamma + 1`` tokens followed by a partial commit is the rollback
of the rejected positions.

Reference counterparts: cg_speculative_decoder / cg_speculative_generate / cg_draft_generate /
cg_target_verify (include/cg_speculative.h:30-112, generate/step/draft/verify declared only),
cg_matmul_int4 and cg_kv_cache_int4_* (src/quantize/int4.c:90-289).
"""
from __future__ import annotations

import os
import warnings
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.llama import Llama, LlamaConfig
from ..ops import _lib
from ..ops import misc as M
from ..ops.attention import flash_forward
from ..ops.norm import rms_norm
from ..quant.int4 import Int4Linear, dequantize_int4, quantize_int4
from .kv_cache import PagedKVCacheInt4
from .sampling import sample, spec_accept


class LlamaInt4Engine:
    """``tp_group``: a process group over which the engine is tensor parallel.  Every rank is given
    the full model and keeps its slice: q/k/v heads and the gate/up columns are split (column
    parallel), the attention output and down projections take the matching input slice (row
    parallel) and their partial results are summed over the group; the vocabulary projection
    is split into 128-aligned slices whose logits are gathered.  The slices are cut before
    quantisation on group boundaries, so every rank holds exactly the values the unsplit engine
    holds and the sampled tokens agree on all ranks (same Philox stream).  Steps of up to ``ar_tokens``
    tokens per sequence use the fused all-reduce + residual + RMSNorm kernel over peer memory; longer
    ones (prompts) fall back to the process group's all-reduce."""

    def __init__(self, model: Llama, batch: int, max_seq_len: int | None = None, weight_group: int = 128,
                 kv_group: int = 32, page_size: int = 64, tp_group=None, ar_tokens: int = 64):
        cfg: LlamaConfig = model.cfg
        self.cfg = cfg
        dev = model.wte.device
        self.device = dev
        self.dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.tp_group = tp_group
        self.tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        r = self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        tp, D, d = self.tp, cfg.head_dim, cfg.d_model
        if cfg.n_head % tp or cfg.n_kv_head % tp:
            raise ValueError("heads and kv heads must be divisible by the tensor-parallel size")
        self.Hq, self.Hk = cfg.n_head // tp, cfg.n_kv_head // tp
        # The MLP's hidden units are dealt out in blocks of the quantisation group, so that every
        # rank's slices are cut on group boundaries (Llama-7B: 11008 = 86 blocks of 128, which 8
        # ranks share as 11, 11, 11, 11, 11, 11, 10, 10).
        if tp > 1:
            if cfg.d_ff % weight_group or cfg.d_ff // weight_group < tp:
                raise ValueError(f"d_ff must be a multiple of the weight group ({weight_group}) with at least one block per rank")
            base, extra = divmod(cfg.d_ff // weight_group, tp)
            ff0 = (r * base + min(r, extra)) * weight_group
            ff = (base + (1 if r < extra else 0)) * weight_group
        else:
            ff0, ff = 0, cfg.d_ff
        nq, nk = cfg.n_head * D, cfg.n_kv_head * D

        def rows(w, *spans):                    # concatenation of row ranges [start, start + n) of a [out, in] weight
            return torch.cat([w[s:s + n] for s, n in spans], 0) if tp > 1 else w

        self.wte = model.wte.detach().to(self.dtype)
        self.layers = []
        for blk in model.blocks:
            qkv_w, gu_w = blk.attn.qkv.weight.data, blk.mlp.gate_up.weight.data
            qkv = rows(qkv_w, (r * self.Hq * D, self.Hq * D), (nq + r * self.Hk * D, self.Hk * D), (nq + nk + r * self.Hk * D, self.Hk * D))
            gate_up = rows(gu_w, (ff0, ff), (cfg.d_ff + ff0, ff))
            proj = blk.attn.proj.weight.data[:, r * self.Hq * D:(r + 1) * self.Hq * D] if tp > 1 else blk.attn.proj.weight.data
            down = blk.mlp.down.weight.data[:, ff0:ff0 + ff] if tp > 1 else blk.mlp.down.weight.data
            self.layers.append(dict(
                norm1=blk.norm1.weight.detach().to(self.dtype), norm2=blk.norm2.weight.detach().to(self.dtype),
                qkv=Int4Linear(qkv, None, weight_group), proj=Int4Linear(proj, None, weight_group),
                gate_up=Int4Linear(gate_up, None, weight_group), down=Int4Linear(down, None, weight_group)))
        self.norm_f = model.norm_f.weight.detach().to(self.dtype)
        V = cfg.vocab_size
        if tp > 1:
            # 128-aligned vocabulary slices, the last one zero-padded; the padding is cut after the gather
            self.v_slice = (V + tp * 128 - 1) // (tp * 128) * 128
            lo, hi = min(V, r * self.v_slice), min(V, (r + 1) * self.v_slice)
            head = torch.zeros(self.v_slice, d, dtype=model.lm_head.weight.dtype, device=dev)
            head[:hi - lo] = model.lm_head.weight.data[lo:hi]
            self.lm_head = Int4Linear(head, None, weight_group)
        else:
            self.lm_head = Int4Linear.from_linear(model.lm_head, weight_group)
        self.max_seq_len = max_seq_len or cfg.max_seq_len
        self.cache = PagedKVCacheInt4(cfg.n_layer, batch, self.max_seq_len, self.Hk, cfg.head_dim, kv_group,
                                      page_size, dev)
        self.rope = M.rope_tables(self.max_seq_len, cfg.head_dim, cfg.rope_theta, dev)
        self.batch = batch
        if tp > 1:
            from ..parallel.serve_comm import ServeAllReduce
            self.ar = ServeAllReduce(tp_group, dev, max_rows=batch * ar_tokens, cols=d)
        self._fresh = True                     # nothing committed since the last reset

    # ------------------------------------------------------------ quantised checkpoints
    _LINEARS = ("qkv", "proj", "gate_up", "down")

    def save(self, path: str) -> int:
        """Writes this rank's engine (embedding and norms in bf16 / fp32, every projection as a packed
        INT4 entry followed by its ``.scales`` entry) as one COG1 file; ``load`` reads it back without
        the full-precision model.  A tensor-parallel engine writes its own slices: one file per rank."""
        from ..io.checkpoint import save_tensors
        t, shapes = {"wte": self.wte, "norm_f": self.norm_f}, {}

        def put(name, lin):
            t[name], t[name + ".scales"] = lin.packed, lin.scales
            shapes[name] = (lin.in_features, lin.out_features)

        for i, l in enumerate(self.layers):
            t[f"layers.{i}.norm1"], t[f"layers.{i}.norm2"] = l["norm1"], l["norm2"]
            for k in self._LINEARS:
                put(f"layers.{i}.{k}", l[k])
        put("lm_head", self.lm_head)
        return save_tensors(path, {k: v.detach().cpu() for k, v in t.items()}, int4_shapes=shapes)

    @classmethod
    def load(cls, path: str, cfg: LlamaConfig, batch: int, device="cpu", max_seq_len: int | None = None, weight_group: int = 128,
             kv_group: int = 32, page_size: int = 64) -> "LlamaInt4Engine":
        """An unsplit engine from a file written by ``save`` (same configuration and weight group)."""
        from ..io.checkpoint import load_tensors
        st = load_tensors(path)
        dev = torch.device(device)
        self = cls.__new__(cls)
        self.cfg, self.device = cfg, dev
        self.dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.tp_group, self.tp, self.tp_rank = None, 1, 0
        self.Hq, self.Hk = cfg.n_head, cfg.n_kv_head
        D, d, ff = cfg.head_dim, cfg.d_model, cfg.d_ff
        shape = {"qkv": (d, (cfg.n_head + 2 * cfg.n_kv_head) * D), "proj": (cfg.n_head * D, d), "gate_up": (d, 2 * ff), "down": (ff, d)}

        def lin(name, in_f, out_f):
            return Int4Linear.from_packed(st[name], st[name + ".scales"], in_f, out_f, weight_group).to(dev)

        self.wte = st["wte"].to(dev, self.dtype)
        self.norm_f = st["norm_f"].to(dev, self.dtype)
        self.layers = [dict(norm1=st[f"layers.{i}.norm1"].to(dev, self.dtype), norm2=st[f"layers.{i}.norm2"].to(dev, self.dtype),
                            **{k: lin(f"layers.{i}.{k}", *shape[k]) for k in cls._LINEARS}) for i in range(cfg.n_layer)]
        self.lm_head = lin("lm_head", d, cfg.vocab_size)
        self.max_seq_len = max_seq_len or cfg.max_seq_len
        self.cache = PagedKVCacheInt4(cfg.n_layer, batch, self.max_seq_len, self.Hk, D, kv_group, page_size, dev)
        self.rope = M.rope_tables(self.max_seq_len, D, cfg.rope_theta, dev)
        self.batch = batch
        self._fresh = True
        return self

    def weight_bytes(self) -> int:
        n = 0
        for l in self.layers:
            for k in ("qkv", "proj", "gate_up", "down"):
                n += l[k].packed.numel() + l[k].scales.numel() * 4
        return n + self.lm_head.packed.numel() + self.lm_head.scales.numel() * 4

    def reset(self):
        self.cache.reset()
        self._fresh = True

    def _proj_add_norm(self, lin: Int4Linear, inp: torch.Tensor, x: torch.Tensor, norm_w: torch.Tensor) -> torch.Tensor:
        """x += (sum over the tensor-parallel ranks of) lin(inp), in place; returns rmsnorm(x) * norm_w.
        With several ranks the projection writes into symmetric memory and one kernel does the sum over
        the peers, the residual add and the norm."""
        rows = x.shape[0] * x.shape[1]
        if self.tp > 1 and rows <= self.ar.max_rows:
            lin(inp.reshape(rows, -1), out=self.ar.slot(rows))
            return self.ar.reduce_add(x.view(rows, -1), rows, norm_w, self.cfg.norm_eps).view_as(x)
        y = lin(inp)
        if self.tp > 1:
            dist.all_reduce(y, group=self.tp_group)
        x += y.view_as(x)
        return rms_norm(x, norm_w, self.cfg.norm_eps)

    def _fake_quant(self, t: torch.Tensor) -> torch.Tensor:
        """bf16 [B, T, H, D] -> the values an INT4 cache entry of it dequantises to."""
        g = self.cache.group
        flat = t.float().contiguous()
        packed, scales = quantize_int4(flat, g)
        return dequantize_int4(packed, scales, flat.numel(), g, torch.bfloat16).view(t.shape)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, commit: bool = False) -> torch.Tensor:
        """tokens [batch, Tq] (int) at positions lengths[b] + t -> logits [batch, Tq, V] (fp32)."""
        cfg = self.cfg
        B, Tq = tokens.shape
        Hq, Hk, D = self.Hq, self.Hk, cfg.head_dim                             # this rank's heads
        x = self.wte[tokens.long()]                                            # [B, Tq, d]
        fresh = self._fresh and Tq >= 16 and self.device.type == "cuda" and D in (64, 128)
        self._fresh = False
        positions = self.cache.lengths[:, None] + torch.arange(Tq, device=self.device, dtype=torch.int32)[None]
        h = rms_norm(x, self.layers[0]["norm1"], cfg.norm_eps)
        for i, l in enumerate(self.layers):
            qkv = l["qkv"](h).view(B, Tq, Hq + 2 * Hk, D)
            M.rope_apply_(qkv[:, :, :Hq + Hk], self.rope[0], self.rope[1], positions=positions)
            self.cache.append(i, qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:])
            if fresh:
                # prompt over an empty cache: causal flash attention over the values the cache now
                # holds (K and V pass through the same quantise / dequantise), no history to stream
                kq, vq = (self._fake_quant(qkv[:, :, a:a + Hk]) for a in (Hq, Hq + Hk))
                o = flash_forward(qkv[:, :, :Hq], kq, vq, causal=True)[0]
            else:
                o = self.cache.attention(i, qkv[:, :, :Hq].contiguous())
            h = self._proj_add_norm(l["proj"], o.reshape(B, Tq, Hq * D), x, l["norm2"])
            nxt = self.layers[i + 1]["norm1"] if i + 1 < len(self.layers) else self.norm_f
            h = self._proj_add_norm(l["down"], M.swiglu(l["gate_up"](h)), x, nxt)
        logits = self.lm_head(h)
        if self.tp > 1:
            parts = [torch.empty_like(logits) for _ in range(self.tp)]
            dist.all_gather(parts, logits.contiguous(), group=self.tp_group)
            logits = torch.cat(parts, -1)[..., :cfg.vocab_size]
        logits = logits.float()
        if commit:
            self.cache.commit(Tq)
        return logits


@dataclass
class SpecStats:
    steps: int = 0
    drafted: int = 0
    accepted: int = 0
    generated: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0


class SpeculativeDecoder:
    """Draft ``gamma`` tokens with the small engine, verify them with one pass of the large one,
    accept / correct on the device, commit both caches to the accepted length."""

    def __init__(self, draft: LlamaInt4Engine, target: LlamaInt4Engine, gamma: int = 4, temperature: float = 1.0,
                 top_k: int = 50, top_p: float = 0.9, seed: int = 0, use_graph: bool | None = None):
        if draft.cfg.vocab_size != target.cfg.vocab_size or draft.batch != target.batch:
            raise ValueError("draft and target must share vocabulary and batch size")
        self.draft, self.target, self.gamma = draft, target, gamma
        self.temperature, self.top_k, self.top_p, self.seed = temperature, top_k, top_p, seed
        self.stats = SpecStats()
        dev = target.device
        self._step = torch.zeros(1, dtype=torch.int64, device=dev)
        self._stats_dev = torch.zeros(2, dtype=torch.int32, device=dev)
        # One decoding step is ~200 small kernels; launched from Python the host is several times slower
        # than the device.  On CUDA the whole step (gamma draft passes, verify, accept, cache bookkeeping)
        # is captured once into a CUDA graph and replayed.  Everything the step depends on lives on the
        # device (cache lengths, random-stream counter, the call counter of the fused tensor-parallel
        # all-reduce), so the recorded launches stay valid.  A split engine's graph also records the process
        # group's all-gather of the logits: call close() before destroying the process group (a process that
        # still held such a graph did not leave torch.distributed's shutdown).  COGITO_SERVE_GRAPH=0 turns
        # graphs off.
        env = os.environ.get("COGITO_SERVE_GRAPH", "1") != "0"
        self.use_graph = (dev.type == "cuda" and env) if use_graph is None else use_graph
        self._graph = None
        self._eager_steps = 0

    def close(self):
        """Drops the captured graph (and with it the collectives recorded in it)."""
        self._graph = None
        self._g_out = None
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def _dist(self, logits2d, step, return_probs=True):
        return sample(logits2d, self.temperature, self.top_k, self.top_p, self.seed, step, return_probs=return_probs)

    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        """prompts [batch, L]: fills both caches with L-1 tokens and returns the last token of each
        prompt, which is the first input of the decoding loop."""
        self.draft.reset()
        self.target.reset()
        if prompts.shape[1] > 1:
            self.draft.forward(prompts[:, :-1], commit=True)
            self.target.forward(prompts[:, :-1], commit=True)
        return prompts[:, -1].clone()

    @torch.no_grad()
    def step(self, last: torch.Tensor):
        """last [batch]: newest token of every sequence, not yet in the caches.  Returns
        (n_accepted [batch], out_tokens [batch, gamma + 1]); out_tokens[b, :n+1] extend sequence b."""
        g, B = self.gamma, last.shape[0]
        dev = self.target.device
        V = self.target.cfg.vocab_size
        self._step += 1
        # ---- draft gamma tokens autoregressively
        drafted = torch.empty(B, g, dtype=torch.int32, device=dev)
        q = torch.empty(B, g, V, dtype=torch.float32, device=dev)
        cur = last.view(B, 1)
        base_len = self.draft.cache.lengths.clone()
        for i in range(g):
            logits = self.draft.forward(cur, commit=True)[:, 0]
            tok, probs = self._dist(logits, self._step * 64 + i)
            drafted[:, i], q[:, i] = tok, probs
            cur = tok.view(B, 1)
        # ---- one target pass over [last, d1 .. dg]
        verify_in = torch.cat([last.view(B, 1).to(torch.int32), drafted], 1)
        logits = self.target.forward(verify_in, commit=False)                     # [B, g+1, V]
        _, p = self._dist(logits.view(B * (g + 1), V), self._step * 64 + 32)
        p = p.view(B, g + 1, V)
        # ---- accept / correct; the kernel advances the target lengths by n + 1
        n_acc, out = spec_accept(drafted, q, p, self.seed, self._step, lengths=self.target.cache.lengths, stats=self._stats_dev)
        # the draft cache holds last + d1..d(g-1); keep last + the accepted drafts that it has
        self.draft.cache.lengths.copy_(base_len + torch.minimum(n_acc + 1, torch.full_like(n_acc, g)))
        self._pending_all_accepted = n_acc == g
        return n_acc, out

    @torch.no_grad()
    def step_full(self, last: torch.Tensor):
        """One complete step with nothing decided on the host: ``step``, then the draft pass over d_gamma
        for every sequence (kept only where all drafts were accepted).  Returns (n_accepted, out_tokens,
        next ``last``)."""
        n_acc, out = self.step(last)
        self._catch_up_draft(out, n_acc)
        nxt = out.gather(1, n_acc.long().view(-1, 1)).view(-1)
        return n_acc, out, nxt

    @torch.no_grad()
    def advance(self, last: torch.Tensor):
        """``step_full`` replayed from a CUDA graph when enabled (captured after two eager steps, which
        create every lazily allocated workspace).  The returned tensors are overwritten by the next call."""
        if not self.use_graph:
            return self.step_full(last)
        if self._graph is None:
            if self._eager_steps < 2:
                self._eager_steps += 1
                return self.step_full(last)
            self._g_last = last.clone()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = _lib.launches()
            # The fused all-reduce alternates between two slots by the parity of a HOST call counter, and the
            # choice is frozen into the captured launches; replays alternate correctly only if one step makes an
            # even number of such calls per engine.  Check that, and put the counters back when capture fails.
            reducers = [e.ar for e in (self.draft, self.target) if getattr(e, "ar", None) is not None]
            epochs = [r.epoch for r in reducers]
            try:
                with torch.cuda.graph(graph):
                    self._g_out = self.step_full(self._g_last)
                if any((r.epoch - e0) % 2 for r, e0 in zip(reducers, epochs)):
                    raise RuntimeError("an odd number of fused all-reduce calls per step cannot be replayed")
            except Exception as e:                               # something in the step cannot be captured here
                for r, e0 in zip(reducers, epochs):
                    r.epoch = e0
                warnings.warn(f"decode step not captured ({e!r}); launching it from Python")
                self.use_graph = False
                return self.step_full(last)
            self._graph = graph
            self.graph_launches = _lib.launches() - before      # kernels of this library in one replay
        self._g_last.copy_(last)
        self._graph.replay()
        return self._g_out

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int):
        """Returns a list of per-sequence token lists (prompt + generated) and the statistics."""
        B = prompts.shape[0]
        seqs = [prompts[b].tolist() for b in range(B)]
        last = self.prefill(prompts)
        produced = 0
        while produced < max_new_tokens:
            n_acc, out, nxt = self.advance(last)
            n_host, out_host = n_acc.tolist(), out.tolist()
            for b in range(B):
                seqs[b].extend(out_host[b][:n_host[b] + 1])
            last = nxt.clone()
            self.stats.steps += 1
            self.stats.drafted += self.gamma * B
            self.stats.accepted += sum(n_host)
            produced += min(n_host) + 1
            self.stats.generated += sum(n + 1 for n in n_host)
        return seqs, self.stats

    def _catch_up_draft(self, out, n_acc):
        """Where all gamma drafts were accepted the draft cache lacks d_gamma: run it through
        (for every sequence, at its own position) and keep the result only for those rows."""
        g = self.gamma
        keep = (n_acc == g).to(torch.int32)
        tok = out[:, g - 1].view(-1, 1)
        self.draft.forward(tok, commit=False)
        self.draft.cache.lengths += keep
