"""Paged INT4 key/value cache and attention over it.

Per layer the pool is ``pages[num_pages, page_size, heads, D/2]`` bytes plus fp32 scales
``[num_pages, page_size, heads, D/group]`` (one token's bytes equal the reference layout
``[layers, max_seq, heads, head_dim/2]`` of cg_kv_cache_int4, src/quantize/int4.c:116-145; a
single page of ``max_seq`` tokens reproduces it exactly).  ``lengths`` counts committed tokens
per sequence once, whatever the number of layers (the reference advances it on every
append, src/quantize/int4.c:233).  Rejected speculative tokens are dropped by not advancing
``lengths`` past them.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import Structure, c_int32, c_void_p

import torch

from ..ops import _lib
from ..quant.int4 import _round_half_away


class KvArgs(Structure):
    _fields_ = [("k_pages", c_void_p), ("v_pages", c_void_p), ("k_scales", c_void_p), ("v_scales", c_void_p),
                ("page_table", c_void_p), ("lengths", c_void_p),
                ("batch", c_int32), ("heads", c_int32), ("D", c_int32), ("group", c_int32),
                ("page_size", c_int32), ("max_pages", c_int32)]


class PagedKVCacheInt4:
    def __init__(self, num_layers: int, batch: int, max_seq_len: int, heads: int, head_dim: int, group: int = 32,
                 page_size: int = 64, device="cpu"):
        if head_dim % group or group % 8:
            raise ValueError("group must be a multiple of 8 that divides head_dim")
        self.num_layers, self.batch, self.heads, self.D, self.group = num_layers, batch, heads, head_dim, group
        self.page_size = page_size
        self.max_pages = (max_seq_len + page_size - 1) // page_size
        self.device = torch.device(device)
        n_pages = batch * self.max_pages
        G = head_dim // group
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=self.device)
        self.k_pages = [mk(n_pages, page_size, heads, head_dim // 2, dt=torch.uint8) for _ in range(num_layers)]
        self.v_pages = [mk(n_pages, page_size, heads, head_dim // 2, dt=torch.uint8) for _ in range(num_layers)]
        self.k_scales = [mk(n_pages, page_size, heads, G, dt=torch.float32) for _ in range(num_layers)]
        self.v_scales = [mk(n_pages, page_size, heads, G, dt=torch.float32) for _ in range(num_layers)]
        # identity placement: sequence b owns pages b*max_pages .. ; any permutation works
        self.page_table = torch.arange(n_pages, dtype=torch.int32, device=self.device).view(batch, self.max_pages)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self._scratch = None

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for ts in (self.k_pages, self.v_pages, self.k_scales, self.v_scales) for t in ts)

    def reset(self):
        self.lengths.zero_()

    def commit(self, n_tokens):
        """Advance the lengths (int or per-sequence tensor) after the appended tokens are accepted."""
        self.lengths += n_tokens

    def _args(self, layer: int) -> KvArgs:
        a = KvArgs()
        a.k_pages, a.v_pages = self.k_pages[layer].data_ptr(), self.v_pages[layer].data_ptr()
        a.k_scales, a.v_scales = self.k_scales[layer].data_ptr(), self.v_scales[layer].data_ptr()
        a.page_table, a.lengths = self.page_table.data_ptr(), self.lengths.data_ptr()
        a.batch, a.heads, a.D, a.group = self.batch, self.heads, self.D, self.group
        a.page_size, a.max_pages = self.page_size, self.max_pages
        return a

    # ------------------------------------------------------------------ append
    def append(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor):
        """k_new, v_new: [batch, T, heads, D]; stored at positions lengths[b] .. lengths[b]+T-1."""
        B, T, H, D = k_new.shape
        if (B, H, D) != (self.batch, self.heads, self.D):
            raise ValueError("shape does not match the cache")
        if k_new.is_cuda:
            k_new, v_new = k_new.to(torch.bfloat16).contiguous(), v_new.to(torch.bfloat16).contiguous()
            a = self._args(layer)
            _lib.check(_lib.lib().cgk_kv_int4_append(ctypes.byref(a), k_new.data_ptr(), v_new.data_ptr(), T,
                                                     _lib.stream_ptr()), "cgk_kv_int4_append")
            _lib.count_launch()
            return
        G = D // self.group
        for src, pages, scales in ((k_new, self.k_pages[layer], self.k_scales[layer]), (v_new, self.v_pages[layer], self.v_scales[layer])):
            x = src.to(torch.bfloat16).float().view(B, T, H, G, self.group)
            amax = x.abs().amax(-1)
            s = torch.where(amax < 1e-10, torch.ones_like(amax), amax / 7.0)
            q = _round_half_away(x / s[..., None]).clamp_(-8, 7).to(torch.int16).view(B, T, H, D) & 0xF
            packed = (q[..., 0::2] | (q[..., 1::2] << 4)).to(torch.uint8)
            for b in range(B):
                for t in range(T):
                    pos = int(self.lengths[b]) + t
                    page = int(self.page_table[b, pos // self.page_size])
                    pages[page, pos % self.page_size] = packed[b, t]
                    scales[page, pos % self.page_size] = s[b, t]

    # -------------------------------------------------------------------- read
    def gather(self, layer: int, b: int, length: int):
        """Dequantised (k, v) [length, heads, D] of one sequence (fp32)."""
        out = []
        for pages, scales in ((self.k_pages[layer], self.k_scales[layer]), (self.v_pages[layer], self.v_scales[layer])):
            pos = torch.arange(length, device=self.device)
            page = self.page_table[b, (pos // self.page_size).long()].long()
            raw = pages[page, (pos % self.page_size).long()].to(torch.int16)          # [len, H, D/2]
            q = torch.stack([raw & 0xF, raw >> 4], -1).reshape(length, self.heads, self.D)
            q = torch.where(q >= 8, q - 16, q).float()
            s = scales[page, (pos % self.page_size).long()]                          # [len, H, G]
            out.append(q * s.repeat_interleave(self.group, -1))
        return out

    def attention(self, layer: int, q: torch.Tensor, splits: int = 0) -> torch.Tensor:
        """q: [batch, Tq, Hq, D], the Tq newest tokens (already appended, not yet committed).
        Query t sees keys 0 .. lengths[b] + t."""
        B, Tq, Hq, D = q.shape
        scale = 1.0 / math.sqrt(D)
        if q.is_cuda:
            q = q.to(torch.bfloat16).contiguous()
            if splits <= 0:
                longest = self.max_pages * self.page_size
                splits = max(1, min(32, 296 // max(1, B * self.heads), (longest + 255) // 256))
            L = _lib.lib()
            need = L.cgk_kv_int4_attention_scratch_floats(B, Hq, Tq, D, splits)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=q.device)
            out = torch.empty_like(q)
            a = self._args(layer)
            _lib.check(L.cgk_kv_int4_attention(ctypes.byref(a), q.data_ptr(), out.data_ptr(), Tq, Hq, scale, splits,
                                               self._scratch.data_ptr(), _lib.stream_ptr()), "cgk_kv_int4_attention")
            _lib.count_launch(2)
            return out
        out = torch.empty(B, Tq, Hq, D, dtype=q.dtype)
        rep = Hq // self.heads
        for b in range(B):
            n = int(self.lengths[b]) + Tq
            k, v = self.gather(layer, b, n)
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
            s = torch.einsum("qhd,khd->hqk", q[b].to(torch.bfloat16).float(), k) * scale
            mask = torch.arange(n)[None, :] > (torch.arange(Tq)[:, None] + n - Tq)
            s = s.masked_fill(mask[None], float("-inf"))
            out[b] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).to(q.dtype)
        return out
