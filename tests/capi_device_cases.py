"""Checks of the cg_cuda_* device layer of the C API, written once and run in both of its modes:
host mode on a machine without a GPU (tests/test_capi_device_cpu.py) and device mode on a B200
(tests/test_capi_device_gpu.py).  Every case moves its operands with cg_tensor_to_cuda, computes
with cg_cuda_* and reads the result back with cg_tensor_to_cpu, and compares with numpy in fp32 /
fp64.  Model: the reference's tests/test_cuda.c (init, malloc + memcpy round trip, elementwise,
reductions, a literal matmul, activations, softmax rows)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_bool, c_char, c_float, c_int, c_size_t, c_void_p

import numpy as np

from capi_defs import FP, IP, FlashParams, T, TensorP, borrowed, cg


class DeviceInfo(Structure):
    _fields_ = [("device_id", c_int), ("cc_major", c_int), ("cc_minor", c_int), ("total_memory", c_size_t),
                ("free_memory", c_size_t), ("multiprocessor_count", c_int), ("max_threads_per_block", c_int),
                ("warp_size", c_int), ("shared_memory_per_block", c_size_t), ("device_name", c_char * 256),
                ("is_available", c_bool)]


_DECLARED = False


def D():
    """The library with the device layer's prototypes declared."""
    global _DECLARED
    lib = cg.lib()
    if _DECLARED:
        return lib
    P, I, F, B = TensorP, c_int, c_float, c_bool
    table = {
        "cg_cuda_init": (B,), "cg_cuda_shutdown": (None,), "cg_cuda_is_available": (B,), "cg_cuda_device_mode": (B,),
        "cg_cuda_device_count": (I,), "cg_cuda_get_device_info": (DeviceInfo, I), "cg_cuda_get_device": (I,),
        "cg_cuda_malloc": (c_void_p, c_size_t), "cg_cuda_free": (None, c_void_p),
        "cg_cuda_malloc_host": (c_void_p, c_size_t), "cg_cuda_free_host": (None, c_void_p),
        "cg_cuda_memcpy": (None, c_void_p, c_void_p, c_size_t, I), "cg_cuda_memset": (None, c_void_p, I, c_size_t),
        "cg_cuda_memcpy_async": (None, c_void_p, c_void_p, c_size_t, I, c_void_p),
        "cg_cuda_device_synchronize": (None,), "cg_cuda_stream_synchronize": (None, c_void_p),
        "cg_cuda_get_last_error": (ctypes.c_char_p,), "cg_cuda_clear_error": (None,),
        "cg_cuda_calculate_launch_dims": (None, I, IP, IP),
        "cg_tensor_cuda_new": (P, IP, I, B), "cg_tensor_cuda_zeros": (P, IP, I, B), "cg_tensor_to_cuda": (P, P),
        "cg_tensor_to_cpu": (P, P), "cg_tensor_is_cuda": (B, P), "cg_tensor_free": (None, P),
        "cg_cuda_tensor_scale": (None, P, F, P), "cg_cuda_tensor_pow": (None, P, F, P),
        "cg_cuda_tensor_matmul": (None, P, P, P), "cg_cuda_tensor_bmm": (None, P, P, P), "cg_cuda_tensor_transpose": (None, P, P),
        "cg_cuda_set_matmul_precision": (None, I),
        "cg_cuda_softmax_forward": (None, P, P, I), "cg_cuda_softmax_backward": (None, P, P, P, I),
        "cg_cuda_layernorm_forward": (None, P, P, P, P, P, P, F, I),
        "cg_cuda_layernorm_backward": (None, P, P, P, P, P, P, P, P, I),
        "cg_cuda_rmsnorm_forward": (None, P, P, P, F),
        "cg_flash_attn_params_new": (POINTER(FlashParams), P, P, P, I, F), "cg_flash_attn_params_free": (None, POINTER(FlashParams)),
        "cg_flash_attention_forward_cuda": (None, POINTER(FlashParams)), "cg_flash_attention_backward_cuda": (None, POINTER(FlashParams)),
        "cg_flash_attention_gqa_cuda": (None, POINTER(FlashParams), I),
        "cg_flash_attention_sliding_window_cuda": (None, POINTER(FlashParams), I),
        "cg_flash_attention_paged_cuda": (None, POINTER(FlashParams), IP, I, I),
        "cg_flash_attention_forward_rope_cuda": (None, POINTER(FlashParams), c_void_p, c_void_p, I),
        "cg_rope_forward_cuda": (None, c_void_p, I, I, I, I, c_void_p, c_void_p, I),
        "cg_rope_backward_cuda": (None, c_void_p, I, I, I, I, c_void_p, c_void_p, I),
        "cg_flash_attn_get_tile_sizes": (None, I, I, IP, IP), "cg_flash_attn_estimate_shmem": (c_size_t, I, I, I),
        "cg_flash_attn_check_config": (B, I, I, I, c_size_t), "cg_tensor_live_count": (I,), "cg_last_error": (I,),
    }
    for name in ("add", "sub", "mul", "div"):
        table[f"cg_cuda_tensor_{name}"] = (None, P, P, P)
    for name in ("exp", "log", "sqrt", "abs"):
        table[f"cg_cuda_tensor_{name}"] = (None, P, P)
    for name in ("sum", "mean", "max", "min"):
        table[f"cg_cuda_tensor_{name}"] = (None, P, I, P)
    for name in ("relu", "sigmoid", "tanh", "gelu"):
        table[f"cg_cuda_{name}_forward"] = (None, P, P)
        table[f"cg_cuda_{name}_backward"] = (None, P, P, P)
    for name, (res, *args) in table.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, list(args)
    _DECLARED = True
    return lib


class Dev:
    """A device tensor owned by the test (freed on exit of the with-block that made it)."""

    def __init__(self):
        self.lib, self.live = D(), []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for p in self.live:
            self.lib.cg_tensor_free(p)
        self.live = []

    def put(self, a, requires_grad=False):
        h = T(a, requires_grad)
        p = self.lib.cg_tensor_to_cuda(h._ptr)
        assert p, self.lib.cg_cuda_get_last_error()
        self.live.append(p)
        return p

    def empty(self, *shape):
        arr = (c_int * len(shape))(*shape)
        p = self.lib.cg_tensor_cuda_zeros(arr, len(shape), False)
        assert p
        self.live.append(p)
        return p

    def get(self, p):
        h = self.lib.cg_tensor_to_cpu(p)
        assert h
        out = borrowed(h)
        self.lib.cg_tensor_free(h)
        return out

    def adopt(self, p):
        self.live.append(p)
        return p


def check_clean(lib):
    assert lib.cg_last_error() == 0, lib.cg_cuda_get_last_error()


def case_bringup(lib, expect_device):
    assert lib.cg_cuda_init() and lib.cg_cuda_is_available()
    assert lib.cg_cuda_device_mode() == expect_device
    assert lib.cg_cuda_device_count() >= 1
    info = lib.cg_cuda_get_device_info(lib.cg_cuda_get_device())
    assert info.is_available and info.warp_size == 32 and info.multiprocessor_count >= 1
    if expect_device:
        assert info.cc_major == 10 and info.total_memory > 2 ** 30 and info.shared_memory_per_block >= 48 * 1024
    g, b = c_int(), c_int()
    lib.cg_cuda_calculate_launch_dims(1000, ctypes.byref(g), ctypes.byref(b))
    assert b.value == 256 and g.value == 4
    lib.cg_cuda_calculate_launch_dims(1 << 30, ctypes.byref(g), ctypes.byref(b))
    assert 0 < g.value <= 65535


def case_memory(lib):
    n = 1000
    src = np.arange(n, dtype=np.float32)
    dst = np.zeros(n, dtype=np.float32)
    d = lib.cg_cuda_malloc(4 * n)
    d2 = lib.cg_cuda_malloc(4 * n)
    pin = lib.cg_cuda_malloc_host(4 * n)
    assert d and d2 and pin
    ctypes.memmove(pin, src.ctypes.data, 4 * n)
    lib.cg_cuda_memcpy(d, pin, 4 * n, 0)
    lib.cg_cuda_memcpy_async(d2, d, 4 * n, 2, None)
    lib.cg_cuda_stream_synchronize(None)
    lib.cg_cuda_memcpy(dst.ctypes.data, d2, 4 * n, 1)
    assert np.array_equal(src, dst)
    lib.cg_cuda_memset(d, 0, 4 * n)
    lib.cg_cuda_memcpy(dst.ctypes.data, d, 4 * n, 1)
    assert not dst.any()
    lib.cg_cuda_free(d)
    lib.cg_cuda_free(d2)
    lib.cg_cuda_free_host(pin)
    lib.cg_cuda_device_synchronize()
    check_clean(lib)


def case_elementwise(lib, expect_device):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((37, 129)).astype(np.float32)
    b = (np.abs(rng.standard_normal((37, 129))) + 0.5).astype(np.float32)
    live0 = lib.cg_tensor_live_count()
    with Dev() as dv:
        da, db, do = dv.put(a), dv.put(b), dv.empty(37, 129)
        assert lib.cg_tensor_is_cuda(da) == expect_device
        for name, ref in (("add", a + b), ("sub", a - b), ("mul", a * b), ("div", a / b)):
            getattr(lib, f"cg_cuda_tensor_{name}")(da, db, do)
            np.testing.assert_allclose(dv.get(do), ref, rtol=1e-6, atol=1e-6)
        lib.cg_cuda_tensor_scale(da, 2.5, do)
        np.testing.assert_allclose(dv.get(do), a * 2.5, rtol=1e-6)
        lib.cg_cuda_tensor_exp(da, do)
        np.testing.assert_allclose(dv.get(do), np.exp(a), rtol=2e-6)
        lib.cg_cuda_tensor_abs(da, do)
        np.testing.assert_allclose(dv.get(do), np.abs(a))
        for name, ref in (("log", np.log(b)), ("sqrt", np.sqrt(b))):
            getattr(lib, f"cg_cuda_tensor_{name}")(db, do)
            np.testing.assert_allclose(dv.get(do), ref, rtol=2e-6, atol=1e-6)
        lib.cg_cuda_tensor_pow(db, 1.5, do)
        np.testing.assert_allclose(dv.get(do), b ** 1.5, rtol=1e-5)
        check_clean(lib)
        # a size mismatch is an error, not a launch
        small = dv.empty(3)
        lib.cg_cuda_tensor_add(da, db, small)
        assert lib.cg_last_error() != 0
    assert lib.cg_tensor_live_count() == live0


def case_reductions(lib):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((5, 33, 7)).astype(np.float32)
    with Dev() as dv:
        da, one = dv.put(a), dv.empty(1)
        for name, fn in (("sum", np.sum), ("mean", np.mean), ("max", np.max), ("min", np.min)):
            getattr(lib, f"cg_cuda_tensor_{name}")(da, -1, one)
            np.testing.assert_allclose(dv.get(one)[0], fn(a.astype(np.float64)), rtol=1e-5, atol=1e-5)
            for axis in range(3):
                shape = [s for i, s in enumerate(a.shape) if i != axis]
                out = dv.empty(*shape)
                getattr(lib, f"cg_cuda_tensor_{name}")(da, axis, out)
                np.testing.assert_allclose(dv.get(out), fn(a.astype(np.float64), axis=axis), rtol=1e-5, atol=1e-5)
        check_clean(lib)
