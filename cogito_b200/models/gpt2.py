"""GPT-2-shaped decoder (learned positions, LayerNorm, GELU MLP, tied output
embedding) built from the framework's transformer block.

Default sizes are GPT-2 small with the vocabulary padded to 50304:
12 layers, d_model 768, 12 heads, MLP 3072, weights N(0, 0.02).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..nn.modules import LayerNorm
from ..nn.transformer import TransformerBlock, TransformerConfig
from ..ops import functional as F
from ..ops import loss as L
from ..ops import misc as M
from ..utils import rng
from ..utils.recompute import checkpoint


@dataclass
class GPT2Config:
    vocab_size: int = 50304
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    d_ff: int = 3072
    max_seq_len: int = 2048
    init_std: float = 0.02
    recompute: bool = False        # drop the activations inside every block and recompute them in backward
    norm_eps: float = 1e-5

    def block_config(self) -> TransformerConfig:
        return TransformerConfig(hidden_size=self.d_model, num_heads=self.n_head, intermediate_size=self.d_ff,
                                 norm_eps=self.norm_eps, bias=True, pre_norm=True, rms_norm=False, swiglu=False,
                                 activation="gelu", causal=True, max_seq_len=self.max_seq_len,
                                 init_std=self.init_std)


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config = GPT2Config(), device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Parameter(rng.normal_(torch.empty(cfg.vocab_size, cfg.d_model, device=device, dtype=dtype),
                                            cfg.init_std, rng.layer_generator()))
        self.wpe = nn.Parameter(rng.normal_(torch.empty(cfg.max_seq_len, cfg.d_model, device=device, dtype=dtype),
                                            cfg.init_std, rng.layer_generator()))
        bc = cfg.block_config()
        self.blocks = nn.ModuleList([TransformerBlock(bc, device, dtype) for _ in range(cfg.n_layer)])
        self.ln_f = LayerNorm(cfg.d_model, cfg.norm_eps, device=device, dtype=dtype)

    def hidden(self, ids: torch.Tensor) -> torch.Tensor:
        x = M.embedding(ids, self.wte, self.wpe)
        for blk in self.blocks:
            x = checkpoint(blk, x) if self.cfg.recompute else blk(x)
        return self.ln_f(x)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor | None = None, grad_scale: float = 1.0):
        """ids: [B, T] int64.  Returns logits [B, T, V], or the mean cross-entropy
        when `targets` is given (its backward yields gradients multiplied by
        `grad_scale`, the loss scale of mixed-precision training)."""
        h = self.hidden(ids)
        logits = F.linear(h, self.wte)
        if targets is None:
            return logits
        return L.cross_entropy(logits, targets, grad_scale)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (forward + backward = 3x forward matmul work,
        causal attention counted at half density)."""
        c = self.cfg
        per_layer = 2 * (3 * c.d_model * c.d_model + c.d_model * c.d_model + 2 * c.d_model * c.d_ff)
        attn = 2 * 2 * seq_len * c.d_model / 2
        head = 2 * c.d_model * c.vocab_size
        return 3.0 * (c.n_layer * (per_layer + attn) + head)
