"""ctypes binding of the host runtime (``libcogito.so``, the ``cg_*`` C API).

``Tensor`` wraps a ``cg_tensor*`` with numpy interop, the eager and tape ops, and
``backward``; ``lib()`` gives the raw library for everything else declared in
``include/cogito.h``.  Counterpart of the reference's ``bindings/cogito.py`` (``CgTensor``,
``Tensor``, ``infer_matmul_shape``), which only covered construction and printing.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_bool, c_char_p, c_float, c_int, c_uint, c_void_p
from pathlib import Path

import numpy as np

CG_MAX_DIMS = 8
CG_MAX_PARENTS = 4


class CgTensor(Structure):
    pass


CgTensor._fields_ = [
    ("data", POINTER(c_float)), ("grad", POINTER(c_float)),
    ("shape", c_int * CG_MAX_DIMS), ("strides", c_int * CG_MAX_DIMS), ("ndim", c_int), ("size", c_int),
    ("requires_grad", c_bool), ("backward_fn", c_void_p),
    ("parents", POINTER(CgTensor) * CG_MAX_PARENTS), ("num_parents", c_int), ("backward_ctx", c_void_p),
    ("ref_count", c_int), ("is_view", c_bool), ("arena", c_void_p),
]
TensorP = POINTER(CgTensor)

_LIB = None


def _find_library() -> str:
    env = os.environ.get("COGITO_LIB")
    if env:
        return env
    here = Path(__file__).resolve().parent
    for cand in (here.parent / "cogito_b200" / "lib" / "libcogito.so", here / "libcogito.so"):
        if cand.exists():
            return str(cand)
    raise OSError("libcogito.so not found: run `python -m cogito_b200.build --capi` or set COGITO_LIB")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(_find_library())
        shape_t = POINTER(c_int)
        for name in ("cg_tensor_new", "cg_tensor_zeros", "cg_tensor_ones"):
            getattr(L, name).restype = TensorP
            getattr(L, name).argtypes = [shape_t, c_int, c_bool]
        L.cg_tensor_randn.restype = TensorP
        L.cg_tensor_randn.argtypes = [shape_t, c_int, c_uint, c_bool]
        L.cg_tensor_from_data.restype = TensorP
        L.cg_tensor_from_data.argtypes = [POINTER(c_float), shape_t, c_int, c_bool]
        L.cg_tensor_release.argtypes = [TensorP]
        L.cg_tensor_retain.argtypes = [TensorP]
        L.cg_tensor_print.argtypes = [TensorP, c_char_p]
        L.cg_tensor_zero_grad.argtypes = [TensorP]
        for name in ("cg_add", "cg_sub", "cg_mul", "cg_matmul"):
            getattr(L, name).restype = TensorP
            getattr(L, name).argtypes = [TensorP, TensorP]
        for name in ("cg_sum_all", "cg_mean_all", "cg_exp", "cg_log_op"):
            getattr(L, name).restype = TensorP
            getattr(L, name).argtypes = [TensorP]
        L.cg_pow_op.restype = TensorP
        L.cg_pow_op.argtypes = [TensorP, c_float]
        L.cg_backward.argtypes = [TensorP]
        L.cg_last_error.restype = c_int
        L.cg_error_string.restype = c_char_p
        L.cg_error_string.argtypes = [c_int]
        L.cg_tensor_live_count.restype = c_int
        L.cg_manual_seed.argtypes = [c_uint]
        _LIB = L
    return _LIB


_DEVICE_READY = False


def _device_lib() -> ctypes.CDLL:
    """The library with the device layer declared and brought up (``cg_cuda_init``: device mode on
    a machine with a GPU and the kernel library beside libcogito.so, host mode otherwise)."""
    global _DEVICE_READY
    L = lib()
    if not _DEVICE_READY:
        for name in ("cg_tensor_to_cuda", "cg_tensor_to_cpu"):
            getattr(L, name).restype, getattr(L, name).argtypes = TensorP, [TensorP]
        L.cg_tensor_cuda_zeros.restype, L.cg_tensor_cuda_zeros.argtypes = TensorP, [POINTER(c_int), c_int, c_bool]
        L.cg_tensor_is_cuda.restype, L.cg_tensor_is_cuda.argtypes = c_bool, [TensorP]
        L.cg_cuda_tensor_matmul.restype, L.cg_cuda_tensor_matmul.argtypes = None, [TensorP, TensorP, TensorP]
        L.cg_cuda_init.restype = c_bool
        L.cg_cuda_device_mode.restype = c_bool
        L.cg_cuda_get_last_error.restype = c_char_p
        L.cg_cuda_init()
        _DEVICE_READY = True
    return L


def device_mode() -> bool:
    """True when ``cg_cuda_*`` calls execute on a GPU, False when they compute on the host."""
    return bool(_device_lib().cg_cuda_device_mode())


def _check(ptr, what: str):
    if not ptr:
        L = lib()
        raise RuntimeError(f"{what}: {L.cg_error_string(L.cg_last_error()).decode()}")
    return ptr


def _shape_arg(shape):
    shape = tuple(int(s) for s in shape)
    if len(shape) > CG_MAX_DIMS:
        raise ValueError(f"at most {CG_MAX_DIMS} dimensions")
    return (c_int * max(len(shape), 1))(*shape), len(shape)


class Tensor:
    """Owns one reference to a ``cg_tensor``."""

    def __init__(self, shape=None, requires_grad: bool = False, _ptr=None):
        if _ptr is not None:
            self._ptr = _ptr
        else:
            arr, n = _shape_arg(shape)
            self._ptr = _check(lib().cg_tensor_zeros(arr, n, requires_grad), "cg_tensor_zeros")

    def __del__(self):
        ptr, self._ptr = getattr(self, "_ptr", None), None
        if ptr and _LIB is not None:
            _LIB.cg_tensor_release(ptr)

    # -- construction
    @staticmethod
    def from_ptr(ptr, retain: bool = False) -> "Tensor":
        if retain:
            lib().cg_tensor_retain(ptr)
        return Tensor(_ptr=ptr)

    @staticmethod
    def from_numpy(a, requires_grad: bool = False) -> "Tensor":
        a = np.ascontiguousarray(a, dtype=np.float32)
        arr, n = _shape_arg(a.shape)
        p = lib().cg_tensor_from_data(a.ctypes.data_as(POINTER(c_float)), arr, n, requires_grad)
        return Tensor(_ptr=_check(p, "cg_tensor_from_data"))

    @staticmethod
    def randn(shape, seed: int = 0, requires_grad: bool = False) -> "Tensor":
        arr, n = _shape_arg(shape)
        return Tensor(_ptr=_check(lib().cg_tensor_randn(arr, n, seed, requires_grad), "cg_tensor_randn"))

    # -- views of the C storage (valid while this object lives)
    @property
    def shape(self):
        c = self._ptr.contents
        return tuple(c.shape[i] for i in range(c.ndim))

    @property
    def requires_grad(self) -> bool:
        return bool(self._ptr.contents.requires_grad)

    def numpy(self) -> np.ndarray:
        c = self._ptr.contents
        return np.ctypeslib.as_array(c.data, shape=(c.size,)).reshape(self.shape)

    @property
    def grad(self):
        c = self._ptr.contents
        if not c.grad:
            return None
        return np.ctypeslib.as_array(c.grad, shape=(c.size,)).reshape(self.shape)

    # -- device layer (cg_cuda_*): device memory on a machine with a GPU, host memory otherwise
    def cuda(self) -> "Tensor":
        """A copy in device memory (``numpy()`` of it is invalid; bring it back with ``cpu()``)."""
        L = _device_lib()
        return Tensor(_ptr=_check(L.cg_tensor_to_cuda(self._ptr), "cg_tensor_to_cuda"))

    def cpu(self) -> "Tensor":
        L = _device_lib()
        return Tensor(_ptr=_check(L.cg_tensor_to_cpu(self._ptr), "cg_tensor_to_cpu"))

    @property
    def is_cuda(self) -> bool:
        return bool(_device_lib().cg_tensor_is_cuda(self._ptr))

    def device_matmul(self, other: "Tensor") -> "Tensor":
        """``cg_cuda_tensor_matmul`` of two device tensors ([M,K] x [K,N]): the tcgen05 GEMM on a B200."""
        L = _device_lib()
        arr, n = _shape_arg((self.shape[0], other.shape[1]))
        out = Tensor(_ptr=_check(L.cg_tensor_cuda_zeros(arr, n, False), "cg_tensor_cuda_zeros"))
        L.cg_cuda_tensor_matmul(self._ptr, other._ptr, out._ptr)
        err = L.cg_last_error()
        if err:
            raise RuntimeError(f"cg_cuda_tensor_matmul: {L.cg_error_string(err).decode()}: {L.cg_cuda_get_last_error().decode()}")
        return out

    def zero_grad(self):
        lib().cg_tensor_zero_grad(self._ptr)

    def print(self, name: str = "tensor"):
        lib().cg_tensor_print(self._ptr, name.encode())

    # -- tape ops
    def _binary(self, other, fn):
        if not isinstance(other, Tensor):
            other = Tensor.from_numpy(np.asarray(other, dtype=np.float32).reshape(-1) if np.ndim(other) else np.array([other], np.float32))
        return Tensor(_ptr=_check(fn(self._ptr, other._ptr), fn.__name__))

    def __add__(self, o): return self._binary(o, lib().cg_add)
    def __sub__(self, o): return self._binary(o, lib().cg_sub)
    def __mul__(self, o): return self._binary(o, lib().cg_mul)
    def __matmul__(self, o): return self._binary(o, lib().cg_matmul)
    def __pow__(self, p): return Tensor(_ptr=_check(lib().cg_pow_op(self._ptr, float(p)), "cg_pow_op"))
    def sum(self): return Tensor(_ptr=_check(lib().cg_sum_all(self._ptr), "cg_sum_all"))
    def mean(self): return Tensor(_ptr=_check(lib().cg_mean_all(self._ptr), "cg_mean_all"))
    def exp(self): return Tensor(_ptr=_check(lib().cg_exp(self._ptr), "cg_exp"))
    def log(self): return Tensor(_ptr=_check(lib().cg_log_op(self._ptr), "cg_log_op"))

    def backward(self):
        lib().cg_backward(self._ptr)

    def __repr__(self):
        return f"Tensor(shape={self.shape}, requires_grad={self.requires_grad})"


def infer_matmul_shape(shape_a, shape_b):
    """Result shape of ``a @ b`` with broadcast leading dimensions; dimensions may be ints
    or names (strings) for symbolic sizes, which must then match by name."""
    a, b = list(shape_a), list(shape_b)
    if len(a) < 2 or len(b) < 2:
        raise ValueError("matmul needs at least 2-D operands")
    if a[-1] != b[-2]:
        raise ValueError(f"inner dimensions differ: {a[-1]} vs {b[-2]}")
    la, lb = a[:-2], b[:-2]
    n = max(len(la), len(lb))
    la, lb = [1] * (n - len(la)) + la, [1] * (n - len(lb)) + lb
    lead = []
    for x, y in zip(la, lb):
        if x == 1:
            lead.append(y)
        elif y == 1 or x == y:
            lead.append(x)
        else:
            raise ValueError(f"leading dimensions do not broadcast: {x} vs {y}")
    return tuple(lead + [a[-2], b[-1]])
