"""The allocation-free column-sum entry point.

Some users of the kernel library cannot allocate device memory when they call it
(a host that gave all GPU memory to its own arena, a latency-critical loop that
must not enter the allocator), so ``cgk_colsum_bf16_noalloc`` keeps its scratch
inside the library.  This test calls it through its exported C symbol, twice in a
row, and checks each result against the ordinary entry point (which takes
caller-provided scratch) within the tolerance used for the other reductions."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from cogito_b200.ops import _lib
    L = _lib.lib()
    fn = L.cgk_colsum_bf16_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return _lib, L, fn


def _reference(_lib, L, x):
    M, N = x.shape
    out = torch.empty(N, device=x.device, dtype=torch.float32)
    scratch = torch.empty(max(1, L.cgk_colsum_scratch_elems(M, N)), device=x.device, dtype=torch.float32)
    _lib.check(L.cgk_colsum_bf16(x.data_ptr(), M, N, x.stride(0), out.data_ptr(), scratch.data_ptr(), 0,
                                 _lib.stream_ptr()))
    return out


def test_no_alloc_colsum_matches_regular_entry_point_twice():
    _l, L, fn = _lib()
    torch.manual_seed(0)
    dev = "cuda"
    # two different shapes back to back: the second call finds the first call's
    # partial sums in the shared scratch and must not be affected by them
    shapes = [(5000, 3000), (777, 100)]
    xs = [torch.randn(M, N, device=dev).to(torch.bfloat16) for M, N in shapes]
    outs = [torch.full((N,), 7.0, device=dev, dtype=torch.float32) for _, N in shapes]
    for x, out in zip(xs, outs):
        rc = fn(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), 0, _l.stream_ptr())
        assert rc == 0, L.cgk_last_error().decode()
    torch.cuda.synchronize()
    for x, out in zip(xs, outs):
        ref = _reference(_l, L, x)
        err = ((out - ref).abs().max() / (ref.abs().max() + 1e-6)).item()
        assert err < 1e-3, err
        exact = x.float().sum(0)
        assert ((out - exact).abs().max() / (exact.abs().max() + 1e-6)).item() < 1e-3
    # accumulate flag
    acc = outs[1].clone()
    assert fn(xs[1].data_ptr(), 777, 100, xs[1].stride(0), acc.data_ptr(), 1, _l.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert ((acc - 2 * outs[1]).abs().max() / (outs[1].abs().max() + 1e-6)).item() < 1e-3


def test_no_alloc_colsum_rejects_oversize():
    _l, L, fn = _lib()
    x = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), 8, 16385, 16385, out.data_ptr(), 0, _l.stream_ptr())
    assert rc == -3
    assert b"16384" in L.cgk_last_error()
