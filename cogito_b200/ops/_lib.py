"""ctypes binding of ``libcogito_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`cogito_b200.build`.  On a machine with a
GPU a missing library is an error, never a silent fallback: every CUDA op of the
package goes through :func:`lib`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_longlong, c_void_p, c_ulonglong
from pathlib import Path

import torch

# COGITO_KERNELS_DEBUG=1 selects the index-checking build (python -m cogito_b200.build --debug-bounds)
_DEBUG = os.environ.get("COGITO_KERNELS_DEBUG", "0") not in ("", "0")
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / ("libcogito_kernels_dbg.so" if _DEBUG else "libcogito_kernels.so")
_lib = None
# source files that carry index checks in the debug build (one recorded violation each)
_BOUNDS_FILES = ("gemm_tcgen05", "softmax_ce", "serving", "elementwise", "flash_fwd", "flash_bwd")


class KernelError(RuntimeError):
    """A kernel launcher returned a non-zero code."""


class GemmArgs(Structure):
    """Mirror of ``cgk_gemm_args`` (include/cogito_kernels.h)."""

    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("out", c_void_p),
        ("M", c_int32), ("N", c_int32), ("K", c_int32), ("batch", c_int32),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("strideA", c_int64), ("strideB", c_int64), ("strideC", c_int64),
        ("a_mn", c_int32), ("b_mn", c_int32),
        ("out_fp32", c_int32), ("accumulate", c_int32),
        ("alpha", c_float),
        ("bias", c_void_p), ("bias_fp32", c_int32), ("act", c_int32),
        ("residual", c_void_p), ("ldr", c_int64),
        ("aux_out", c_void_p), ("ldaux", c_int64),
        ("aux_in", c_void_p), ("ldauxin", c_int64),
        ("dact", c_int32), ("force_simt", c_int32), ("max_ctas", c_int32),
        ("rope_cos", c_void_p), ("rope_sin", c_void_p),
        ("rope_cols", c_int32), ("rope_D", c_int32), ("rope_T", c_int32), ("rope_pos0", c_int32), ("rope_inverse", c_int32),
        ("split_k", c_int32),
    ]


def _declare(L: ctypes.CDLL) -> None:
    vp, i, f, ll = c_void_p, c_int, c_float, c_longlong
    L.cgk_last_error.restype = c_char_p
    L.cgk_version.restype = c_int
    L.cgk_read_status.argtypes = [POINTER(c_int), vp]
    L.cgk_gemm_bf16.argtypes = [POINTER(GemmArgs), vp]
    sigs = {
        "cgk_norm_forward": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, f, i, vp],
        "cgk_norm_backward": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, vp],
        "cgk_softmax_ce_fused": [vp, vp, vp, vp, i, i, ll, f, vp, ll, vp],
        "cgk_ce_stats": [vp, vp, ll, vp, vp, vp, i, i, ll, vp],
        "cgk_ce_backward": [vp, vp, ll, vp, vp, i, i, ll, f, vp, ll, vp],
        "cgk_softmax_rows": [vp, vp, i, i, f, vp],
        "cgk_softmax_rows_backward": [vp, vp, vp, i, i, vp],
        "cgk_softmax_dropout_residual": [i, vp, vp, vp, vp, i, i, f, c_ulonglong, vp],
        "cgk_softmax_dropout_residual_backward": [i, vp, vp, vp, vp, i, i, f, c_ulonglong, vp],
        "cgk_scaler_init": [vp, f, vp],
        "cgk_grad_stats": [vp, ll, vp, vp, i, vp],
        "cgk_adam_step": [vp, vp, vp, vp, vp, ll, f, f, f, f, f, f, vp, vp],
        "cgk_sgd_step": [vp, vp, vp, vp, ll, f, f, f, i, f, vp, vp],
        "cgk_scaler_update": [vp, f, f, i, f, f, vp],
        "cgk_binary": [i, i, vp, vp, vp, ll, i, POINTER(c_int), POINTER(c_longlong), POINTER(c_longlong), vp],
        "cgk_unary": [i, i, vp, vp, ll, f, vp],
        "cgk_unary_backward": [i, i, vp, vp, vp, ll, f, vp],
        "cgk_cast": [vp, vp, ll, i, vp],
        "cgk_reduce_axis": [i, i, vp, vp, ll, ll, ll, vp],
        "cgk_reduce_all": [i, i, vp, ll, vp, vp, vp],
        "cgk_colsum_bf16": [vp, ll, i, ll, vp, vp, i, vp],
        "cgk_embedding_forward": [vp, vp, vp, vp, ll, i, i, ll, ll, vp],
        "cgk_embedding_backward": [vp, vp, vp, vp, ll, i, i, ll, ll, vp],
        "cgk_dropout": [i, vp, vp, ll, f, c_ulonglong, vp],
        "cgk_swiglu_forward": [i, vp, vp, ll, i, vp],
        "cgk_swiglu_backward": [i, vp, vp, vp, ll, i, vp],
        "cgk_transpose2d": [i, vp, vp, i, i, vp],
        "cgk_batchnorm_forward": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, f, f, i, vp],
        "cgk_batchnorm_backward": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp],
        "cgk_im2col": [i, vp, vp, i, i, i, i, i, i, i, i, i, ll, vp],
        "cgk_col2im": [i, vp, vp, i, i, i, i, i, i, i, i, i, ll, vp],
        "cgk_maxpool_forward": [vp, vp, vp, i, i, i, i, i, i, i, i, vp],
        "cgk_maxpool_backward": [vp, vp, vp, i, i, i, i, i, i, vp],
        "cgk_rope_table": [vp, vp, i, i, f, vp],
        "cgk_rope_apply": [i, vp, vp, vp, vp, i, i, i, i, ll, ll, ll, i, i, i, vp],
        "cgk_int4_quantize": [vp, ll, i, vp, vp, vp],
        "cgk_int4_dequantize": [vp, vp, ll, i, vp, vp, vp],
        "cgk_int4_gemm": [vp, ll, vp, vp, vp, vp, ll, vp, i, i, i, i, vp],
        "cgk_int4_tile_weights": [vp, vp, i, i, i, vp, vp],
        "cgk_int4_wa_gemm": [vp, ll, vp, vp, vp, vp, ll, vp, i, i, i, i, vp],
        "cgk_int4_wa_tile_weights": [vp, vp, i, i, i, vp, vp],
        "cgk_kv_int4_append": [vp, vp, vp, i, vp],
        "cgk_kv_int4_attention": [vp, vp, vp, i, i, f, i, vp, vp],
        "cgk_sample": [vp, i, ll, i, i, f, i, f, c_ulonglong, vp, vp, vp, vp],
        "cgk_spec_accept": [vp, vp, vp, i, i, i, c_ulonglong, vp, vp, vp, vp, vp, vp],
        "cgk_tree_mask": [vp, i, i, vp, vp, vp],
    }
    for name, argtypes in sigs.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = c_int
    for name, argtypes in {
        "cgk_norm_backward_scratch_elems": [i, i],
        "cgk_colsum_scratch_elems": [ll, i],
        "cgk_kv_int4_attention_scratch_floats": [i, i, i, i, i],
        "cgk_int4_tiles_bytes": [i, i],
        "cgk_int4_wa_tiles_bytes": [i, i],
        "cgk_int4_gemm_counters": [i, i],
    }.items():
        fn = getattr(L, name)
        fn.argtypes = argtypes
        fn.restype = c_longlong
    L.cgk_grad_stats_scratch_elems.argtypes = [ll]
    L.cgk_reduce_all_scratch_elems.argtypes = [ll]
    L.cgk_scaler_state_bytes.argtypes = []


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """The loaded kernel library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python -m cogito_b200.build` (needs nvcc). "
                "CUDA tensors cannot be processed without it."
            )
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().cgk_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what or 'kernel call'} failed (code {rc}): {msg}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def read_status() -> tuple[int, int, int, int]:
    """Synchronise the current stream and return (code, where, block, aux) of the
    device status word; code 0 means no kernel reported a problem."""
    out = (c_int * 4)()
    check(lib().cgk_read_status(out, stream_ptr()), "cgk_read_status")
    return tuple(out)  # type: ignore[return-value]


def read_bounds(reset: bool = True) -> list[tuple[str, int, int, int]]:
    """Index violations recorded by the debug build: (source file, line, index, limit); empty with the
    ordinary library.  Synchronises."""
    if not _DEBUG:
        return []
    torch.cuda.synchronize()
    out = []
    for name in _BOUNDS_FILES:
        fn = getattr(lib(), f"cgk_bounds_read_{name}", None)
        if fn is None:
            continue
        word = (c_int * 4)()
        if fn(word, int(reset)) == 0 and word[0] != 0:
            out.append((name, word[1], word[2], word[3]))
    return out


def assert_device_ok() -> None:
    code, where, block, aux = read_status()
    if code != 0:
        raise KernelError(f"device status: code={code} where={where} block={block} aux={aux}")
    bad = read_bounds()
    if bad:
        raise KernelError(f"index outside its range (file, line, index, limit): {bad}")


# ---------------------------------------------------------------------------
# Gradient slots.  A parameter's fp32 gradient buffer is ``p.main_grad``.  A model that runs two
# parts of a batch on two streams at once gives every parameter one buffer per part
# (``p.main_grad_slots``) so that the two backward passes never accumulate into the same memory
# concurrently; autograd Functions note the slot that was current in their forward pass and
# select it again around their backward pass.
# ---------------------------------------------------------------------------
_grad_slot = 0


def grad_slot() -> int:
    return _grad_slot


def set_grad_slot(i: int) -> int:
    """Selects the gradient slot; returns the previous one."""
    global _grad_slot
    prev, _grad_slot = _grad_slot, int(i)
    return prev


def main_grad_of(p):
    """The fp32 buffer the gradient of ``p`` is accumulated into (None: use autograd's .grad)."""
    if p is None:
        return None
    slots = getattr(p, "main_grad_slots", None)
    if slots is not None:
        return slots[_grad_slot]
    return getattr(p, "main_grad", None)


_launches = 0


def count_launch(n: int = 1) -> None:
    """Launch accounting used by bench.py (kernels of this library only)."""
    global _launches
    _launches += n


def launches() -> int:
    return _launches


def reset_launches() -> None:
    global _launches
    _launches = 0
