"""Batched sampling, speculative accept/correct/commit, tree-attention masks.

GPU: ``cgk_sample`` / ``cgk_spec_accept`` / ``cgk_tree_mask`` (csrc/kernels/serving.cu).
CPU: the same composition in PyTorch — temperature, then top-k, then top-p, then renormalise —
which is also the oracle of the GPU tests.  The reference has the three samplers as separate
functions (src/inference/speculative.c:54-146) and the acceptance rule
``min(1, p_target / p_draft)`` with residual resampling (``:49, :148-172``).
"""
from __future__ import annotations

import torch

from ..ops import _lib

MAX_TOPK = 1024


def filtered_probs(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """fp32 [rows, V] distribution after temperature -> top-k -> top-p (host restatement)."""
    x = logits.float()
    V = x.shape[-1]
    if temperature <= 0:
        return torch.nn.functional.one_hot(x.argmax(-1), V).float()
    x = x / temperature
    k = MAX_TOPK if top_k <= 0 or top_k > MAX_TOPK else top_k
    k = min(k, V)
    # descending by value, smaller index first among ties (what the kernel's sort does)
    order = torch.argsort(-x, dim=-1, stable=True)[..., :k]
    vals = torch.gather(x, -1, order)
    p = torch.softmax(vals, -1)
    if 0.0 < top_p < 1.0:
        csum = torch.cumsum(p, -1)
        keep = (csum - p) < top_p            # the first token always stays; stop once the mass is reached
        p = p * keep
    p = p / p.sum(-1, keepdim=True)
    return torch.zeros_like(x).scatter_(-1, order, p)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           step: torch.Tensor | int = 0, return_probs: bool = False, generator: torch.Generator | None = None):
    """logits [rows, V] -> tokens int32 [rows] (and the fp32 [rows, V] distribution sampled from)."""
    rows, V = logits.shape
    if logits.is_cuda:
        logits = logits.contiguous()
        if logits.dtype not in (torch.float32, torch.bfloat16):
            logits = logits.float()
        tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
        probs = torch.empty(rows, V, dtype=torch.float32, device=logits.device) if return_probs else None
        if not isinstance(step, torch.Tensor):
            step = torch.tensor([int(step)], dtype=torch.int64, device=logits.device)
        _lib.check(_lib.lib().cgk_sample(logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), rows, V,
                                         float(temperature), int(top_k), float(top_p), int(seed), step.data_ptr(),
                                         tokens.data_ptr(), _lib.ptr(probs), _lib.stream_ptr()), "cgk_sample")
        _lib.count_launch()
        return (tokens, probs) if return_probs else tokens
    probs = filtered_probs(logits, temperature, top_k, top_p)
    if generator is None:
        generator = torch.Generator().manual_seed(int(seed) * 1000003 + int(step))
    tokens = torch.multinomial(probs, 1, generator=generator).view(-1).to(torch.int32)
    return (tokens, probs) if return_probs else tokens


def spec_accept(draft_tokens: torch.Tensor, q: torch.Tensor, p: torch.Tensor, seed: int = 0, step: torch.Tensor | int = 0,
                lengths: torch.Tensor | None = None, stats: torch.Tensor | None = None,
                generator: torch.Generator | None = None):
    """draft_tokens [B, g] int32; q [B, g, V] draft distributions; p [B, g+1, V] target
    distributions.  Returns (n_accepted [B], out_tokens [B, g+1]); out_tokens[b, :n+1] are the
    tokens to append.  ``lengths`` (int32 [B]) is advanced by n+1; ``stats`` (int32 [2]) accumulates
    (drafted, accepted)."""
    B, g = draft_tokens.shape
    V = q.shape[-1]
    if draft_tokens.is_cuda:
        draft_tokens = draft_tokens.to(torch.int32).contiguous()
        q, p = q.float().contiguous(), p.float().contiguous()
        n_acc = torch.empty(B, dtype=torch.int32, device=q.device)
        out = torch.zeros(B, g + 1, dtype=torch.int32, device=q.device)
        if not isinstance(step, torch.Tensor):
            step = torch.tensor([int(step)], dtype=torch.int64, device=q.device)
        _lib.check(_lib.lib().cgk_spec_accept(draft_tokens.data_ptr(), q.data_ptr(), p.data_ptr(), B, g, V, int(seed),
                                              step.data_ptr(), n_acc.data_ptr(), out.data_ptr(), _lib.ptr(lengths),
                                              _lib.ptr(stats), _lib.stream_ptr()), "cgk_spec_accept")
        _lib.count_launch()
        return n_acc, out
    if generator is None:
        generator = torch.Generator().manual_seed(int(seed) * 7919 + int(step) + 1)
    n_acc = torch.zeros(B, dtype=torch.int32)
    out = torch.zeros(B, g + 1, dtype=torch.int32)
    for b in range(B):
        n = 0
        while n < g:
            tok = int(draft_tokens[b, n])
            pd, pt = float(q[b, n, tok]), float(p[b, n, tok])
            ratio = min(1.0, pt / pd) if pd > 0 else 1.0
            if not (float(torch.rand((), generator=generator)) < ratio):
                break
            out[b, n] = tok
            n += 1
        resid = p[b, n].float() if n == g else (p[b, n].float() - q[b, n].float()).clamp_min(0)
        if float(resid.sum()) <= 1e-12:
            resid = p[b, n].float()
        out[b, n] = int(torch.multinomial(resid / resid.sum(), 1, generator=generator))
        n_acc[b] = n
    if lengths is not None:
        lengths += n_acc + 1
    if stats is not None:
        stats[0] += B * g
        stats[1] += int(n_acc.sum())
    return n_acc, out


def tree_attention_mask(parents: torch.Tensor, prefix_len: int, dtype=torch.float32) -> torch.Tensor:
    """parents int32 [n] (-1 = child of the prefix) -> additive mask [L+n, L+n] of 0 / -1e9."""
    n = parents.numel()
    T = prefix_len + n
    if parents.is_cuda:
        parents = parents.to(torch.int32).contiguous()
        mask = torch.empty(T, T, dtype=dtype, device=parents.device)
        f32 = mask.data_ptr() if dtype == torch.float32 else None
        b16 = mask.data_ptr() if dtype == torch.bfloat16 else None
        _lib.check(_lib.lib().cgk_tree_mask(parents.data_ptr(), n, prefix_len, f32, b16, _lib.stream_ptr()), "cgk_tree_mask")
        _lib.count_launch()
        return mask
    vis = torch.zeros(T, T, dtype=torch.bool)
    vis[:prefix_len, :prefix_len] = torch.tril(torch.ones(prefix_len, prefix_len, dtype=torch.bool))
    vis[prefix_len:, :prefix_len] = True
    for i in range(n):
        a = i
        while a >= 0:
            vis[prefix_len + i, prefix_len + a] = True
            a = int(parents[a])
    return torch.where(vis, 0.0, -1e9).to(dtype)
