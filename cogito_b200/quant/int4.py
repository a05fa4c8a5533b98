"""INT4 weight quantisation and the weight-only GEMM that consumes it.

Format (bit-exact with cg_quantize_int4, src/quantize/int4.c:10-59): flat groups of
``group`` consecutive elements of the row-major tensor, ``scale = absmax / 7`` (1 when below
1e-10), ``q = clamp(round(x / scale), -8, 7)`` with halves rounded away from zero, two values
per byte with the even index in the low nibble, fp32 scales.

``Int4Linear`` keeps the weight transposed, ``[in, out]`` like the reference's
``cg_matmul_int4`` operand (src/quantize/int4.c:90-114), so that the tcgen05 kernel streams
each weight row once; on CPU the same product is computed from the dequantised weight.
"""
from __future__ import annotations

import os

import torch

from ..ops import _lib


def _round_half_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(torch.abs(x) + 0.5)


def quantize_int4(x: torch.Tensor, group: int = 128):
    """Returns (packed uint8 [ceil(n/2)], scales fp32 [ceil(n/group)]) of the flattened tensor."""
    if group <= 0 or group % 2:
        raise ValueError("group must be a positive even number")
    flat = x.detach().reshape(-1).float().contiguous()
    n = flat.numel()
    groups = (n + group - 1) // group
    if flat.is_cuda:
        packed = torch.zeros((n + 1) // 2, dtype=torch.uint8, device=flat.device)
        scales = torch.empty(groups, dtype=torch.float32, device=flat.device)
        _lib.check(_lib.lib().cgk_int4_quantize(flat.data_ptr(), n, group, packed.data_ptr(), scales.data_ptr(),
                                                _lib.stream_ptr()), "cgk_int4_quantize")
        _lib.count_launch()
        return packed, scales
    pad = groups * group - n
    g = torch.nn.functional.pad(flat, (0, pad)).view(groups, group)
    amax = g.abs().amax(1)
    scales = torch.where(amax < 1e-10, torch.ones_like(amax), amax / 7.0)
    q = _round_half_away(g / scales[:, None]).clamp_(-8, 7).to(torch.int16).view(-1)[:n + (n & 1)]
    if q.numel() < n + (n & 1):
        q = torch.nn.functional.pad(q, (0, n + (n & 1) - q.numel()))
    q = q & 0xF
    packed = (q[0::2] | (q[1::2] << 4)).to(torch.uint8)
    return packed, scales


def dequantize_int4(packed: torch.Tensor, scales: torch.Tensor, n: int, group: int = 128,
                    dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if packed.is_cuda:
        out = torch.empty(n, dtype=dtype, device=packed.device)
        f32 = out.data_ptr() if dtype == torch.float32 else None
        b16 = out.data_ptr() if dtype == torch.bfloat16 else None
        if f32 is None and b16 is None:
            raise ValueError("dtype must be float32 or bfloat16")
        _lib.check(_lib.lib().cgk_int4_dequantize(packed.data_ptr(), scales.data_ptr(), n, group, f32, b16,
                                                  _lib.stream_ptr()), "cgk_int4_dequantize")
        _lib.count_launch()
        return out
    b = packed.to(torch.int16)
    q = torch.stack([b & 0xF, b >> 4], 1).reshape(-1)[:n]
    q = torch.where(q >= 8, q - 16, q).float()
    idx = torch.arange(n) // group
    return (q * scales[idx]).to(dtype)


class Int4Linear(torch.nn.Module):
    """y = x @ W^T (+ bias) with W stored as packed INT4 of W^T ([in, out], groups along out)."""

    # Which tcgen05 kernel multiplies: "wb" keeps the weights as the B operand (converted tile in shared
    # memory, 128 token rows per instruction), "wa" makes them the A operand fed from tensor memory (cost
    # follows the token count; needs group % 128 == 0).  "auto": "wa" up to 32 token rows, where it measured
    # faster, "wb" above.  Each kernel has its own tile-major copy of the weights, made on first use.
    kernel = os.environ.get("COGITO_INT4_KERNEL", "auto")

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, group: int = 128):
        super().__init__()
        out_f, in_f = weight.shape
        if out_f % group:
            raise ValueError(f"out_features {out_f} must be a multiple of the group size {group}")
        self.in_features, self.out_features, self.group = in_f, out_f, group
        packed, scales = quantize_int4(weight.detach().t().contiguous(), group)
        self.register_buffer("packed", packed)
        self.register_buffer("scales", scales)
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.bfloat16))
        self._acc = None
        self._tiles = {}                      # kernel kind -> tile-major weights

    @classmethod
    def from_packed(cls, packed: torch.Tensor, scales: torch.Tensor, in_features: int, out_features: int, group: int = 128,
                    bias: torch.Tensor | None = None) -> "Int4Linear":
        """Wraps already quantised values (of W^T, [in, out] row-major, as ``quantize_int4`` returns them),
        e.g. read from a checkpoint; nothing is re-quantised."""
        if packed.numel() != (in_features * out_features + 1) // 2 or scales.numel() != (in_features * out_features + group - 1) // group:
            raise ValueError("packed / scales do not match the layer shape and group size")
        self = cls.__new__(cls)
        torch.nn.Module.__init__(self)
        self.in_features, self.out_features, self.group = in_features, out_features, group
        self.register_buffer("packed", packed.to(torch.uint8).contiguous())
        self.register_buffer("scales", scales.to(torch.float32).contiguous())
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.bfloat16))
        self._acc = None
        self._tiles = {}
        return self

    @classmethod
    def from_linear(cls, lin, group: int = 128) -> "Int4Linear":
        return cls(lin.weight.data, getattr(lin, "bias", None), group)

    def dequantized(self, dtype=torch.float32) -> torch.Tensor:
        """W^T as [in, out]."""
        return dequantize_int4(self.packed, self.scales, self.in_features * self.out_features, self.group, dtype) \
            .view(self.in_features, self.out_features)

    def forward(self, x: torch.Tensor, splits: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
        """``out``: an optional contiguous [rows, out_features] buffer for the result (bf16 on CUDA),
        e.g. a slot of symmetric memory that a collective kernel reads next."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        M = x2.shape[0]

        def done(y):
            if out is None:
                return y.view(*lead, self.out_features)
            out.copy_(y.view(out.shape))
            return out.view(*lead, self.out_features)

        if not x2.is_cuda:
            y = x2.float() @ self.dequantized()
            if self.bias is not None:
                y = y + self.bias.float()
            return done(y.to(x.dtype))
        N, K = self.out_features, self.in_features
        if N % 128 or K % 64 or self.group % 64:
            # shapes the streaming kernel does not cover: dequantise once, then the bf16 GEMM
            from ..ops.gemm import gemm
            w = self.dequantized(torch.bfloat16)
            return done(gemm(x2.to(torch.bfloat16).contiguous(), w, b_mn=True, bias=self.bias))
        x2 = x2.to(torch.bfloat16).contiguous()
        L = _lib.lib()
        # "wa": weights on the M side of the tensor core (needs one scale per k for a 128-feature tile)
        wa = (self.kernel == "wa" or (self.kernel == "auto" and M <= 32)) and self.group % 128 == 0 and K % 128 == 0
        tiles = self._tiles.get(wa)
        if tiles is None or tiles.device != x2.device:
            # one-time tile-major reordering of the same quantised values
            nbytes, tile = (L.cgk_int4_wa_tiles_bytes, L.cgk_int4_wa_tile_weights) if wa else (L.cgk_int4_tiles_bytes, L.cgk_int4_tile_weights)
            tiles = self._tiles[wa] = torch.empty(nbytes(K, N), dtype=torch.uint8, device=x2.device)
            _lib.check(tile(self.packed.data_ptr(), self.scales.data_ptr(), K, N, self.group,
                            tiles.data_ptr(), _lib.stream_ptr()), "cgk_int4_tile_weights")
            _lib.count_launch()
        if self._acc is None or self._acc.numel() < M * N or self._acc.device != x2.device:
            # split-K scratch: zero once, every call leaves it zero again
            self._acc = torch.zeros(M * N, dtype=torch.float32, device=x2.device)
            self._counters = torch.zeros(L.cgk_int4_gemm_counters(M, N), dtype=torch.int32, device=x2.device)
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)
        elif out.dtype != torch.bfloat16 or not out.is_contiguous() or out.numel() != M * N:
            raise ValueError("out must be a contiguous bf16 [rows, out_features] tensor")
        _lib.check((L.cgk_int4_wa_gemm if wa else L.cgk_int4_gemm)(
            x2.data_ptr(), K, tiles.data_ptr(), self._acc.data_ptr(), self._counters.data_ptr(),
            out.data_ptr(), N, _lib.ptr(self.bias), M, N, K, splits, _lib.stream_ptr()), "cgk_int4_gemm")
        _lib.count_launch()
        return out.view(*lead, N)
