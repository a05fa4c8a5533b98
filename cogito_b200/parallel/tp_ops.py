"""Fused tensor-parallel primitives: all-gather -> GEMM and GEMM -> reduce-scatter,
each ONE kernel (``cgk_ag_gemm`` / ``cgk_gemm_rs``, csrc/comm/fused_tp.cu).

``TPWorkspace`` owns the symmetric memory the kernels need: the activation-shard
buffer and the handshake words of the all-gather, and the double-buffered partial-product
buffers (each rank writes its own, the owners of the rows read them over NVLink) and arrival
counters of the reduce-scatter.  CPU tensors (gloo ranks, or one
rank) take a reference path built from ``torch.distributed`` collectives, which is
also the oracle of the GPU tests.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_int32, c_int64, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import _ld, fill_rope, gemm
from .symm import SymmetricBuffer


class AgArgs(Structure):
    _fields_ = [("rank", c_int32), ("ranks", c_int32), ("epoch", c_int32), ("chunk_rows", c_int32),
                ("shard_ptrs", c_void_p * 8), ("signal_ptrs", c_void_p * 8),
                ("chunk_flag_ptrs", c_void_p * 8), ("done_count", c_void_p), ("n_copy_ctas", c_int32),
                ("mc_gathered", c_void_p)]


class RsArgs(Structure):
    _fields_ = [("rank", c_int32), ("ranks", c_int32), ("queue_base", c_int32),
                ("partial_ptrs", c_void_p * 8), ("flag_ptrs", c_void_p * 8),
                ("ld", c_int64), ("bias", c_void_p), ("residual", c_void_p),
                ("ldr", c_int64), ("out", c_void_p), ("ldo", c_int64), ("n_reduce_ctas", c_int32),
                ("queue", c_void_p), ("mc_partial", c_void_p)]


_declared = False


def _fns():
    global _declared
    L = _lib.lib()
    if not _declared:
        L.cgk_ag_gemm.argtypes = [POINTER(_lib.GemmArgs), POINTER(AgArgs), c_void_p]
        L.cgk_gemm_rs.argtypes = [POINTER(_lib.GemmArgs), POINTER(RsArgs), c_void_p]
        L.cgk_gemm_rs_queue_step.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        _declared = True
    return L


class TPWorkspace:
    """Symmetric scratch of one tensor-parallel group on one device.

    max_rows: largest M (gathered rows) of any call; max_cols: largest K of an
    all-gather / N of a reduce-scatter.

    When the symmetric-memory provider bound the buffers to an NVSwitch multicast object
    (and ``COGITO_TP_NVLS`` is not ``0``) the kernels use it: the reduce-scatter sums inside
    the switch, and the all-gather is a multicast store, for which the gathered activations
    must live in symmetric memory themselves.  ``arena_bytes`` reserves that memory: gathered
    buffers that outlive the call (saved for the backward pass) are carved from it one after
    the other and all released together by :meth:`begin_step`, which the model calls at the
    start of every forward pass; two more buffers alternate for gathers whose result is
    consumed at once.  A request that does not fit falls back to the peer-load kernel and
    an ordinary tensor."""

    def __init__(self, device, group=None, max_rows: int = 16384, max_cols: int = 4096,
                 chunk_rows: int = 256, copy_ctas: int = 0, reduce_ctas: int = 0, max_ctas: int = 0,
                 arena_bytes: int = 0):
        self.device = torch.device(device)
        self.group = group
        self.ranks = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        P = self.ranks
        self.max_rows, self.max_cols, self.chunk_rows = max_rows, max_cols, chunk_rows
        self.copy_ctas, self.reduce_ctas, self.max_ctas = copy_ctas, reduce_ctas, max_ctas
        self.cuda = self.device.type == "cuda"
        self.epoch = 0
        self.parity = 0
        self.nvls = False
        self.arena = None
        if not self.cuda or P == 1:
            return
        shard_rows = (max_rows + P - 1) // P
        self.shard_bytes = shard_rows * max_cols * 2
        self.sig_off = (self.shard_bytes + 255) // 256 * 256
        sig_bytes = 256
        self.slot_elems = shard_rows * max_cols
        self.stage_off = self.sig_off + sig_bytes
        stage_bytes = 2 * P * self.slot_elems * 2
        self.flag_off = (self.stage_off + stage_bytes + 255) // 256 * 256
        self.flag_words = (shard_rows + 127) // 128
        flag_bytes = (2 * self.flag_words * 4 + 255) // 256 * 256
        # chunk flags of the all-gather: written locally (peer-load mode) or by the rank that
        # multicast the chunk; one word per 128 rows is enough for any chunk size
        self.cflag_off = self.flag_off + flag_bytes
        cflag_bytes = (((max_rows + 127) // 128 + P) * 4 + 255) // 256 * 256
        self.buf = SymmetricBuffer(self.cflag_off + cflag_bytes, self.device, group)
        self.shard = self.buf.view(0, (self.shard_bytes,), torch.uint8)
        self.done_count = torch.zeros(P, dtype=torch.int32, device=self.device)
        self.rs_queue = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.rs_queue_base = 0
        self.nvls = bool(self.buf.multicast_ptr) and os.environ.get("COGITO_TP_NVLS", "1") not in ("", "0")
        self.transient_bytes = (max_rows * max_cols * 2 + 255) // 256 * 256
        self.arena_pos = 0
        self._transient = 0
        if self.nvls:
            self.arena = SymmetricBuffer(2 * self.transient_bytes + max(0, int(arena_bytes)), self.device, group)
            if not self.arena.multicast_ptr:
                self.arena = None
        self.begin_step()

    # ------------------------------------------------------------------
    def shard_view(self, rows: int, cols: int) -> torch.Tensor:
        return self.buf.view(0, (rows, cols), torch.bfloat16)

    def begin_step(self) -> None:
        """Releases every gathered buffer handed out since the last call (they are overwritten
        by the next forward pass)."""
        if self.arena is not None:
            self.arena_pos = 2 * self.transient_bytes

    def alloc_gathered(self, rows: int, cols: int, keep: bool):
        """(tensor [rows, cols] bf16 in the multicast arena, its multicast address), or None."""
        if self.arena is None:
            return None
        nbytes = (rows * cols * 2 + 255) // 256 * 256
        if keep:
            if self.arena_pos + nbytes > self.arena.nbytes:
                return None
            off = self.arena_pos
            self.arena_pos += nbytes
        else:
            if nbytes > self.transient_bytes:
                return None
            off = self._transient * self.transient_bytes
            self._transient ^= 1
        return self.arena.view(off, (rows, cols), torch.bfloat16), self.arena.multicast_ptr + off


def _fill_gemm(g, a, b, out, M, N, K, b_mn):
    g.A, g.B = a.data_ptr(), b.data_ptr()
    g.out = out.data_ptr() if out is not None else a.data_ptr()
    g.M, g.N, g.K, g.batch = M, N, K, 1
    g.lda, g.ldb = _ld(a), _ld(b)
    g.ldc = _ld(out) if out is not None else N
    g.a_mn, g.b_mn = 0, int(b_mn)
    g.alpha = 1.0


def ag_gemm(ws: TPWorkspace, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False,
            bias=None, act=None, aux_out=None, aux_in=None, dact=None, out_dtype=torch.bfloat16,
            keep: bool = True, rope=None):
    """Returns (out [M, N], gathered [M, K]) with M = ranks * x_shard.shape[0].

    out = act(gather(x_shard) @ W^T + bias) [* dact'(aux_in)]; ``w`` is [N, K] (or [K, N] with
    b_mn).  ``keep=False`` says that the gathered matrix is consumed before the next-but-one
    gather (it may then sit in one of the two alternating multicast buffers).  ``rope``: rotary
    specification for the GEMM's epilogue (see ``ops.gemm.gemm``)."""
    rows, K = x_shard.shape
    P = ws.ranks
    M = rows * P
    N = w.shape[1] if b_mn else w.shape[0]
    if not x_shard.is_cuda:
        if P > 1:
            parts = [torch.empty_like(x_shard) for _ in range(P)]
            dist.all_gather(parts, x_shard.contiguous(), group=ws.group)
            gathered = torch.cat(parts, 0)
        else:
            gathered = x_shard
        out = gemm(gathered, w, b_mn=b_mn, bias=bias, act=act, aux_out=aux_out, aux_in=aux_in, dact=dact,
                   out_dtype=out_dtype, rope=rope)
        return out, gathered
    if P == 1:
        x_shard = x_shard.contiguous()
        return gemm(x_shard, w, b_mn=b_mn, bias=bias, act=act, aux_out=aux_out, aux_in=aux_in, dact=dact,
                    out_dtype=out_dtype, rope=rope), x_shard
    if rows % 128 or K % 8:
        raise ValueError("ag_gemm: rows per rank must be a multiple of 128 and K of 8")
    x_shard = x_shard.contiguous()
    mc = ws.alloc_gathered(M, K, keep) if ws.nvls else None
    if mc is not None:
        gathered, mc_addr = mc
    else:
        if rows * K * 2 > ws.shard_bytes:
            raise ValueError("ag_gemm: shard larger than the workspace")
        # the shard must sit in symmetric memory for the peers to read it
        sv = ws.shard_view(rows, K)
        if x_shard.data_ptr() != sv.data_ptr():
            sv.copy_(x_shard)
        gathered, mc_addr = torch.empty(M, K, device=x_shard.device, dtype=torch.bfloat16), None
    out = torch.empty(M, N, device=x_shard.device, dtype=out_dtype)
    g = _lib.GemmArgs()
    _fill_gemm(g, gathered, w, out, M, N, K, b_mn)
    g.out_fp32 = int(out_dtype == torch.float32)
    if bias is not None:
        g.bias, g.bias_fp32 = bias.data_ptr(), int(bias.dtype == torch.float32)
    g.act = {"none": 0, None: 0, "gelu": 1, "relu": 2, "silu": 3, "sigmoid": 4, "tanh": 5}[act]
    if aux_out is not None:
        g.aux_out, g.ldaux = aux_out.data_ptr(), _ld(aux_out)
    if aux_in is not None:
        g.aux_in, g.ldauxin = aux_in.data_ptr(), _ld(aux_in)
        g.dact = {"none": 0, None: 0, "gelu": 1, "relu": 2, "silu": 3, "sigmoid": 4, "tanh": 5}[dact]
    g.max_ctas = ws.max_ctas
    if rope is not None:
        fill_rope(g, rope, x_shard.device)
    ws.epoch += 1
    a = AgArgs()
    a.rank, a.ranks, a.epoch = ws.rank, P, ws.epoch
    chunk = min(ws.chunk_rows, rows)
    a.chunk_rows = chunk
    for r, p in enumerate(ws.buf.peer_ptrs(0)):
        a.shard_ptrs[r] = p
    if mc_addr is not None:
        a.shard_ptrs[ws.rank] = x_shard.data_ptr()      # read locally, broadcast through the switch
        a.mc_gathered = mc_addr
    for r, p in enumerate(ws.buf.peer_ptrs(ws.sig_off)):
        a.signal_ptrs[r] = p
    for r, p in enumerate(ws.buf.peer_ptrs(ws.cflag_off)):
        a.chunk_flag_ptrs[r] = p
    a.done_count = ws.done_count.data_ptr()
    a.n_copy_ctas = ws.copy_ctas
    _lib.check(_fns().cgk_ag_gemm(ctypes.byref(g), ctypes.byref(a), _lib.stream_ptr()), "cgk_ag_gemm")
    _lib.count_launch()
    return out, gathered


def gemm_rs(ws: TPWorkspace, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None,
            residual=None):
    """out_shard [M/ranks, N] = bias + residual + rows-of-this-rank( sum_p x_p @ W_p^T ).

    ``x``: this rank's [M, K_local]; ``w``: [N, K_local] (or [K_local, N] with b_mn)."""
    M, K = x.shape
    P = ws.ranks
    N = w.shape[1] if b_mn else w.shape[0]
    rows = M // P
    if not x.is_cuda:
        partial = gemm(x, w, b_mn=b_mn, out_dtype=torch.float32 if x.dtype == torch.bfloat16 else x.dtype)
        if P > 1:
            partial = partial.to(x.dtype).float()       # the kernel ships bf16 partials
            parts = list(partial.chunk(P, 0))
            mine = torch.empty_like(parts[0])
            dist.reduce_scatter(mine, [p.contiguous() for p in parts], group=ws.group)
        else:
            mine = partial.float()
        if bias is not None:
            mine = mine + bias.float()
        if residual is not None:
            mine = mine + residual.float()
        return mine.to(x.dtype)
    if P == 1:
        return gemm(x, w, b_mn=b_mn, bias=bias, residual=residual)
    if M % P or rows % 128 or N % 8:
        raise ValueError("gemm_rs: rows per rank must be a multiple of 128 and N of 8")
    if M * N > P * ws.slot_elems:
        raise ValueError("gemm_rs: partial product larger than the workspace")
    if x.stride(-1) != 1:
        x = x.contiguous()
    out = torch.empty(rows, N, device=x.device, dtype=torch.bfloat16)
    g = _lib.GemmArgs()
    _fill_gemm(g, x, w, None, M, N, K, b_mn)
    r = RsArgs()
    r.rank, r.ranks = ws.rank, P
    par = ws.parity
    ws.parity ^= 1
    stage = ws.stage_off + par * P * ws.slot_elems * 2
    for i, p in enumerate(ws.buf.peer_ptrs(stage)):
        r.partial_ptrs[i] = p
    for i, p in enumerate(ws.buf.peer_ptrs(ws.flag_off + par * ws.flag_words * 4)):
        r.flag_ptrs[i] = p
    r.ld = N
    if bias is not None:
        r.bias = bias.data_ptr()
    if residual is not None:
        r.residual, r.ldr = residual.data_ptr(), _ld(residual)
    r.out, r.ldo = out.data_ptr(), N
    r.n_reduce_ctas = ws.reduce_ctas
    if ws.nvls:
        r.mc_partial = ws.buf.multicast_ptr + stage
    r.queue = ws.rs_queue.data_ptr()
    r.queue_base = ws.rs_queue_base
    g.max_ctas = ws.max_ctas
    ws.rs_queue_base += _fns().cgk_gemm_rs_queue_step(M, P, ws.max_ctas)
    if ws.rs_queue_base > 2 ** 30:       # keep the counter far from overflow
        torch.cuda.current_stream().synchronize()
        ws.rs_queue.zero_()
        ws.rs_queue_base = 0
    _lib.check(_fns().cgk_gemm_rs(ctypes.byref(g), ctypes.byref(r), _lib.stream_ptr()), "cgk_gemm_rs")
    _lib.count_launch()
    return out
