"""Second half of the device-layer checks (see capi_device_cases.py): matrix products,
activations and their gradients, softmax, normalisations, attention and RoPE."""
from __future__ import annotations

import ctypes
from ctypes import c_int

import numpy as np

from capi_device_cases import Dev, check_clean


def _gelu(x):
    return 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))


def case_matmul(lib, expect_device):
    with Dev() as dv:
        # the reference's literal case: [2,3] x [3,2]
        a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
        b = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
        out = dv.empty(2, 2)
        lib.cg_cuda_tensor_matmul(dv.put(a), dv.put(b), out)
        np.testing.assert_allclose(dv.get(out), [[58, 64], [139, 154]], rtol=1e-6)
        # tensor-core sized, odd sized, and batched products against fp64
        rng = np.random.default_rng(2)
        for (M, K, N) in ((256, 512, 384), (100, 70, 36)):
            a = rng.standard_normal((M, K)).astype(np.float32)
            b = rng.standard_normal((K, N)).astype(np.float32)
            ref = a.astype(np.float64) @ b.astype(np.float64)
            out = dv.empty(M, N)
            da, db = dv.put(a), dv.put(b)
            lib.cg_cuda_tensor_matmul(da, db, out)
            err = np.abs(dv.get(out) - ref).max() / np.abs(ref).max()
            assert err < 2e-5, err                       # fp32-class: three bf16 products of split operands
            if expect_device:
                lib.cg_cuda_set_matmul_precision(1)
                lib.cg_cuda_tensor_matmul(da, db, out)
                lib.cg_cuda_set_matmul_precision(3)
                err1 = np.abs(dv.get(out) - ref).max() / np.abs(ref).max()
                assert err < err1 < 2e-2, (err, err1)    # one bf16 product: bf16-class error
        a = rng.standard_normal((3, 64, 128)).astype(np.float32)
        b = rng.standard_normal((3, 128, 64)).astype(np.float32)
        out = dv.empty(3, 64, 64)
        lib.cg_cuda_tensor_bmm(dv.put(a), dv.put(b), out)
        ref = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
        assert np.abs(dv.get(out) - ref).max() / np.abs(ref).max() < 2e-5
        t = dv.empty(128, 64)
        lib.cg_cuda_tensor_transpose(dv.put(a[0]), t)
        np.testing.assert_array_equal(dv.get(t), a[0].T)
        check_clean(lib)


def case_activations(lib):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((50, 40)).astype(np.float32)
    g = rng.standard_normal((50, 40)).astype(np.float32)
    x64 = x.astype(np.float64)
    sig, th = 1 / (1 + np.exp(-x64)), np.tanh(x64)
    eps = 1e-4
    fwd = {"relu": np.maximum(x64, 0), "sigmoid": sig, "tanh": th, "gelu": _gelu(x64)}
    bwd = {"relu": g * (x > 0), "sigmoid": g * sig * (1 - sig), "tanh": g * (1 - th * th),
           "gelu": g * (_gelu(x64 + eps) - _gelu(x64 - eps)) / (2 * eps)}
    with Dev() as dv:
        dx, dg, y, gx = dv.put(x), dv.put(g), dv.empty(50, 40), dv.empty(50, 40)
        for name in ("relu", "sigmoid", "tanh", "gelu"):
            getattr(lib, f"cg_cuda_{name}_forward")(dx, y)
            np.testing.assert_allclose(dv.get(y), fwd[name], rtol=1e-5, atol=1e-6)
            saved = y if name in ("sigmoid", "tanh") else dx          # these two differentiate from the output
            getattr(lib, f"cg_cuda_{name}_backward")(saved, dg, gx)
            np.testing.assert_allclose(dv.get(gx), bwd[name], rtol=1e-4, atol=1e-5)
        check_clean(lib)


def case_softmax(lib):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((6, 10, 33)) * 3).astype(np.float32)
    g = rng.standard_normal((6, 10, 33)).astype(np.float32)
    with Dev() as dv:
        dx, dg, y, gx = dv.put(x), dv.put(g), dv.empty(6, 10, 33), dv.empty(6, 10, 33)
        for axis in (2, -1, 1, 0):
            e = np.exp(x.astype(np.float64) - x.max(axis=axis, keepdims=True))
            ref = e / e.sum(axis=axis, keepdims=True)
            lib.cg_cuda_softmax_forward(dx, y, axis)
            got = dv.get(y)
            np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-7)
            np.testing.assert_allclose(got.sum(axis=axis), 1.0, rtol=1e-5)
            lib.cg_cuda_softmax_backward(y, dg, gx, axis)
            np.testing.assert_allclose(dv.get(gx), ref * (g - (ref * g).sum(axis=axis, keepdims=True)), rtol=1e-4, atol=1e-6)
        check_clean(lib)


def case_norms(lib):
    rng = np.random.default_rng(5)
    rows, Dn = 19, 100                                   # a row length no fused bf16 kernel would take
    x = (rng.standard_normal((rows, Dn)) * 2 + 1).astype(np.float32)
    gamma = rng.standard_normal(Dn).astype(np.float32)
    beta = rng.standard_normal(Dn).astype(np.float32)
    dy = rng.standard_normal((rows, Dn)).astype(np.float32)
    x64 = x.astype(np.float64)
    mu, var = x64.mean(1, keepdims=True), x64.var(1, keepdims=True)
    rs = 1 / np.sqrt(var + 1e-5)
    xhat = (x64 - mu) * rs
    with Dev() as dv:
        dx, dgam, dbet, y = dv.put(x), dv.put(gamma), dv.put(beta), dv.empty(rows, Dn)
        mean, rstd = dv.empty(rows), dv.empty(rows)
        lib.cg_cuda_layernorm_forward(dx, dgam, dbet, y, mean, rstd, 1e-5, Dn)
        np.testing.assert_allclose(dv.get(y), xhat * gamma + beta, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(dv.get(mean), mu[:, 0], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(dv.get(rstd), rs[:, 0], rtol=1e-5)
        gx, ggam, gbet = dv.empty(rows, Dn), dv.empty(Dn), dv.empty(Dn)
        lib.cg_cuda_layernorm_backward(dv.put(dy), dx, dgam, mean, rstd, gx, ggam, gbet, Dn)
        gh = dy.astype(np.float64) * gamma
        ref_dx = rs * (gh - gh.mean(1, keepdims=True) - xhat * (gh * xhat).mean(1, keepdims=True))
        np.testing.assert_allclose(dv.get(gx), ref_dx, rtol=1e-3, atol=1e-5)
        np.testing.assert_allclose(dv.get(ggam), (dy * xhat).sum(0), rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(dv.get(gbet), dy.astype(np.float64).sum(0), rtol=1e-4, atol=1e-4)
        lib.cg_cuda_rmsnorm_forward(dx, dgam, y, 1e-6)
        np.testing.assert_allclose(dv.get(y), x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-6) * gamma, rtol=1e-4, atol=1e-5)
        check_clean(lib)


def _attention(q, k, v, causal=False, window=0):
    """fp64 attention of [B,T,H,D] tensors with grouped KV heads; window: keys at distance < window."""
    B, Tq, H, Dh = q.shape
    Tk, Hk = k.shape[1], k.shape[2]
    kk, vv = np.repeat(k, H // Hk, axis=2).astype(np.float64), np.repeat(v, H // Hk, axis=2).astype(np.float64)
    s = np.einsum("bqhd,bkhd->bhqk", q.astype(np.float64), kk) / np.sqrt(Dh)
    rel = np.arange(Tk)[None, :] - (np.arange(Tq)[:, None] + Tk - Tq)
    if causal or window:
        s = np.where(rel > 0, -np.inf, s)
    if window:
        s = np.where(-rel >= window, -np.inf, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhqk,bkhd->bqhd", p, vv), p


def case_attention(lib, expect_device):
    rng = np.random.default_rng(6)
    B, T, H, Hk, Dh = 2, 128, 4, 2, 64
    q = rng.standard_normal((B, T, H, Dh)).astype(np.float32)
    k = rng.standard_normal((B, T, Hk, Dh)).astype(np.float32)
    v = rng.standard_normal((B, T, Hk, Dh)).astype(np.float32)
    do = rng.standard_normal((B, T, H, Dh)).astype(np.float32)
    tol = 3e-2 if expect_device else 1e-4                # the device kernels compute in bf16
    with Dev() as dv:
        dq, dk, dvv = dv.put(q), dv.put(k), dv.put(v)
        p = lib.cg_flash_attn_params_new(dq, dk, dvv, 1, 0.0)            # causal
        lib.cg_flash_attention_gqa_cuda(p, Hk)
        check_clean(lib)
        ref, _ = _attention(q, k, v, causal=True)
        np.testing.assert_allclose(dv.get(p.contents.O), ref, atol=tol, rtol=tol)
        # backward against a numeric-free closed form: autograd of the fp64 reference by hand
        p.contents.dO = dv.put(do)
        lib.cg_flash_attention_backward_cuda(p)
        check_clean(lib)
        _, P = _attention(q, k, v, causal=True)
        rep = H // Hk
        vv = np.repeat(v, rep, axis=2).astype(np.float64)
        kk = np.repeat(k, rep, axis=2).astype(np.float64)
        dP = np.einsum("bqhd,bkhd->bhqk", do.astype(np.float64), vv)
        dS = P * (dP - (P * dP).sum(-1, keepdims=True)) / np.sqrt(Dh)
        ref_dq = np.einsum("bhqk,bkhd->bqhd", dS, kk)
        ref_dk = np.einsum("bhqk,bqhd->bkhd", dS, q.astype(np.float64)).reshape(B, T, Hk, rep, Dh).sum(3)
        ref_dv = np.einsum("bhqk,bqhd->bkhd", P, do.astype(np.float64)).reshape(B, T, Hk, rep, Dh).sum(3)
        for got, want in ((p.contents.dQ, ref_dq), (p.contents.dK, ref_dk), (p.contents.dV, ref_dv)):
            np.testing.assert_allclose(dv.get(got), want, atol=2 * tol * np.abs(want).max(), rtol=tol)
        # sliding window
        lib.cg_flash_attention_sliding_window_cuda(p, 32)
        check_clean(lib)
        ref, _ = _attention(q, k, v, window=32)
        np.testing.assert_allclose(dv.get(p.contents.O), ref, atol=tol, rtol=tol)
        p.contents.dO = None                                            # owned by the test's Dev
        lib.cg_flash_attn_params_free(p)
        # paged: a shuffled block pool must reproduce the contiguous result
        bs, nblk = 16, B * T // 16
        perm = rng.permutation(nblk)
        pool_k = np.zeros((nblk, bs, Hk, Dh), np.float32)
        pool_v = np.zeros_like(pool_k)
        table = np.zeros((B, T // bs), np.int32)
        for b in range(B):
            for j in range(T // bs):
                blk = perm[b * (T // bs) + j]
                table[b, j] = blk
                pool_k[blk], pool_v[blk] = k[b, j * bs:(j + 1) * bs], v[b, j * bs:(j + 1) * bs]
        p = lib.cg_flash_attn_params_new(dq, dk, dvv, 1, 0.0)
        p.contents.K, p.contents.V = dv.put(pool_k), dv.put(pool_v)     # the block pools take the K / V slots
        lib.cg_flash_attention_paged_cuda(p, table.ctypes.data_as(ctypes.POINTER(c_int)), bs, T)
        check_clean(lib)
        ref, _ = _attention(q, k, v, causal=True)
        np.testing.assert_allclose(dv.get(p.contents.O), ref, atol=tol, rtol=tol)
        lib.cg_flash_attn_params_free(p)


def case_rope(lib):
    rng = np.random.default_rng(7)
    B, T, H, Dh, off = 2, 9, 3, 16, 5
    x = rng.standard_normal((B, T, H, Dh)).astype(np.float32)
    pos = np.arange(off + T)[:, None] * (10000.0 ** (-2.0 * np.arange(Dh // 2) / Dh))[None, :]
    cos, sin = np.cos(pos).astype(np.float32), np.sin(pos).astype(np.float32)
    c, s = cos[off:off + T][None, :, None, :], sin[off:off + T][None, :, None, :]
    x0, x1 = x[..., :Dh // 2], x[..., Dh // 2:]
    ref = np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], -1)
    with Dev() as dv:
        dx, dc, ds = dv.put(x), dv.put(cos), dv.put(sin)
        args = (ctypes.cast(dx.contents.data, ctypes.c_void_p), B, T, H, Dh, ctypes.cast(dc.contents.data, ctypes.c_void_p),
                ctypes.cast(ds.contents.data, ctypes.c_void_p), off)
        lib.cg_rope_forward_cuda(*args)
        np.testing.assert_allclose(dv.get(dx), ref, rtol=1e-5, atol=1e-5)
        lib.cg_rope_backward_cuda(*args)                               # the inverse rotation restores x
        np.testing.assert_allclose(dv.get(dx), x, rtol=1e-5, atol=1e-5)
        check_clean(lib)
    bm, bn = c_int(), c_int()
    lib.cg_flash_attn_get_tile_sizes(128, 100, ctypes.byref(bm), ctypes.byref(bn))
    assert (bm.value, bn.value) == (256, 128)
    need = lib.cg_flash_attn_estimate_shmem(256, 128, 128)
    assert lib.cg_flash_attn_check_config(256, 128, 128, 227 * 1024) == (need <= 227 * 1024)
    assert not lib.cg_flash_attn_check_config(256, 128, 128, 1024)
