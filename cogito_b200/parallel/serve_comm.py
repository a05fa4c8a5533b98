"""Communication of the tensor-parallel serving engine: the sum of a row-parallel projection's
partial results over the ranks, fused with the residual add and the following RMSNorm in one
kernel over NVLink peer memory (``cgk_serve_allreduce``, csrc/comm/serve_allreduce.cu).

The projection writes its partial straight into a slot of symmetric memory (``slot()``), the
kernel reads every rank's slot.  Two slots are used alternately.  On CPU ranks, or with one rank,
the same result is computed with ``torch.distributed.all_reduce``.

Reference counterpart: the all-reduce of cg_tp_row_parallel_forward
(src/pipeline/tensor_parallel.c:81-105).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.norm import rms_norm
from .symm import SymmetricBuffer


class ServeAllReduce:
    def __init__(self, group, device, max_rows: int, cols: int):
        self.group = group
        self.P = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.device = torch.device(device)
        self.max_rows, self.cols = max_rows, cols
        self.epoch = 0
        self.fused = self.P > 1 and self.device.type == "cuda"
        if self.fused:
            if cols % 8 or cols > 16384 or self.P > 8:
                raise ValueError("fused all-reduce: cols must be a multiple of 8 up to 16384, at most 8 ranks")
            self.slot_bytes = (max_rows * cols * 2 + 255) // 256 * 256
            self.buf = SymmetricBuffer(2 * self.slot_bytes + 256, device, group)
            L = _lib.lib()
            L.cgk_serve_allreduce.argtypes = [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]
            L.cgk_serve_allreduce.restype = c_int
            self._fn = L.cgk_serve_allreduce
            self._sig = (c_void_p * self.P)(*self.buf.peer_ptrs(2 * self.slot_bytes))
            self._counters = torch.zeros(2, dtype=torch.int32, device=self.device)   # the kernel numbers its calls here
            self._slots = [(c_void_p * self.P)(*self.buf.peer_ptrs(s * self.slot_bytes)) for s in range(2)]
        else:
            self._local = None

    def slot(self, rows: int) -> torch.Tensor:
        """Where the next partial result [rows, cols] (bf16) has to be written."""
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the workspace ({self.max_rows})")
        if self.fused:
            return self.buf.view(((self.epoch + 1) & 1) * self.slot_bytes, (rows, self.cols), torch.bfloat16)
        if self._local is None or self._local.shape[0] < rows:
            self._local = torch.empty(max(rows, self.max_rows), self.cols, device=self.device,
                                      dtype=torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        return self._local[:rows]

    def reduce_add(self, x: torch.Tensor, rows: int, norm_weight: torch.Tensor | None = None, eps: float = 1e-5):
        """x [rows, cols] += sum over ranks of the partials written into ``slot(rows)``; returns
        rmsnorm(x) * norm_weight (or None without a weight)."""
        self.epoch += 1
        if self.fused:
            h = torch.empty_like(x) if norm_weight is not None else None
            _lib.check(self._fn(self._slots[self.epoch & 1], self._sig, self.rank, self.P, self._counters.data_ptr(), x.data_ptr(),
                                _lib.ptr(norm_weight), _lib.ptr(h), rows, self.cols, eps, _lib.stream_ptr()),
                       "cgk_serve_allreduce")
            _lib.count_launch()
            return h
        part = self._local[:rows]
        if self.P > 1:
            dist.all_reduce(part, group=self.group)
        x += part.to(x.dtype)
        return rms_norm(x, norm_weight, eps) if norm_weight is not None else None
