"""Llama-style decoder: RMSNorm, rotary positions, grouped-query attention, SwiGLU MLP,
no biases, untied output head.

The block is the same ``TransformerBlock`` as GPT-2 with the switches of
cg_transformer_config (include/cg_transformer.h:19-34: ``use_rms_norm``, ``use_swiglu``,
``num_kv_heads``) turned on and RoPE applied inside the packed attention
(src/attention/flash_attn.c:330-365 for the rotation convention: element i pairs with
i + head_dim/2).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..nn.modules import Linear, RMSNorm
from ..nn.transformer import TransformerBlock, TransformerConfig
from ..ops import loss as L
from ..ops import misc as M
from ..utils import rng
from ..utils.recompute import checkpoint


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    n_layer: int = 32
    d_model: int = 4096
    n_head: int = 32
    n_kv_head: int = 8
    d_ff: int = 11008
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    recompute: bool = False        # drop the activations inside every block and recompute them in backward

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    def block_config(self) -> TransformerConfig:
        return TransformerConfig(hidden_size=self.d_model, num_heads=self.n_head, num_kv_heads=self.n_kv_head,
                                 intermediate_size=self.d_ff, norm_eps=self.norm_eps, bias=False, pre_norm=True,
                                 rms_norm=True, swiglu=True, causal=True, rope=True, rope_theta=self.rope_theta,
                                 max_seq_len=self.max_seq_len, init_std=self.init_std)


def llama_7b() -> LlamaConfig:
    return LlamaConfig()


def llama_draft() -> LlamaConfig:
    """Small draft model sharing the 7B vocabulary (speculative decoding)."""
    return LlamaConfig(n_layer=4, d_model=1024, n_head=8, n_kv_head=8, d_ff=2816)


def llama_tiny(vocab_size: int = 256) -> LlamaConfig:
    return LlamaConfig(vocab_size=vocab_size, n_layer=2, d_model=128, n_head=2, n_kv_head=1, d_ff=256, max_seq_len=256)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig = LlamaConfig(), device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Parameter(rng.normal_(torch.empty(cfg.vocab_size, cfg.d_model, device=device, dtype=dtype),
                                            cfg.init_std, rng.layer_generator()))
        bc = cfg.block_config()
        self.blocks = nn.ModuleList([TransformerBlock(bc, device, dtype) for _ in range(cfg.n_layer)])
        self.norm_f = RMSNorm(cfg.d_model, cfg.norm_eps, device=device, dtype=dtype)
        self.lm_head = Linear(cfg.d_model, cfg.vocab_size, bias=False, init_std=cfg.init_std, device=device, dtype=dtype)

    def hidden(self, ids: torch.Tensor) -> torch.Tensor:
        x = M.embedding(ids, self.wte, None)
        for blk in self.blocks:
            x = checkpoint(blk, x) if self.cfg.recompute else blk(x)
        return self.norm_f(x)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor | None = None, grad_scale: float = 1.0):
        logits = self.lm_head(self.hidden(ids))
        if targets is None:
            return logits
        return L.cross_entropy(logits, targets, grad_scale)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq_len: int) -> float:
        c = self.cfg
        kv = c.n_kv_head * c.head_dim
        per_layer = 2 * (c.d_model * (c.d_model + 2 * kv) + c.d_model * c.d_model + 3 * c.d_model * c.d_ff)
        attn = 2 * 2 * seq_len * c.d_model / 2
        return 3.0 * (c.n_layer * (per_layer + attn) + 2 * c.d_model * c.vocab_size)
