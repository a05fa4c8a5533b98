"""Numerics of every CUDA kernel against a plain PyTorch fp32 restatement of the same
op, on small, ragged and boundary shapes.  All tests here need a B200."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def relerr(x, ref):
    x, ref = x.float(), ref.float()
    return ((x - ref).abs().max() / (ref.abs().max() + 1e-6)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    from cogito_b200.ops import _lib
    yield
    _lib.assert_device_ok()


# ---------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 256, 512), (300, 200, 136), (1000, 776, 768),
                                   (4096, 3072, 768), (77, 24, 40)])
@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from cogito_b200.ops.gemm import gemm, gemm_reference
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a leading dimension that is a multiple of 8")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert relerr(out, ref) < 1e-2


@pytest.mark.parametrize("Mw,Nw,K,split", [(384, 768, 16384, 0), (768, 768, 8192, 4), (288, 768, 4096 + 64, 3),
                                           (3072, 768, 2048, 0)])
def test_gemm_split_k_weight_gradient(Mw, Nw, K, split):
    """dW[Mw, Nw] += dy[K, Mw]^T x[K, Nw] in fp32: few output tiles, long reduction, sliced over the SMs."""
    from cogito_b200.ops.gemm import gemm
    torch.manual_seed(2)
    dy = torch.randn(K, Mw, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(K, Nw, device=DEV, dtype=torch.bfloat16)
    base = torch.randn(Mw, Nw, device=DEV, dtype=torch.float32)
    out = base.clone()
    gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True, split_k=split)
    ref = base + dy.float().T @ x.float()
    assert relerr(out, ref) < 2e-3
    one = base.clone()
    gemm(dy, x, a_mn=True, b_mn=True, out=one, accumulate=True, split_k=1)      # unsliced
    assert relerr(one, ref) < 2e-3


@pytest.mark.parametrize("D,heads_rot,heads_all,T", [(64, 6, 9, 128), (128, 5, 6, 96), (64, 3, 3, 64), (128, 2, 3, 50)])
@pytest.mark.parametrize("inverse", [False, True])
def test_gemm_rotary_epilogue(D, heads_rot, heads_all, T, inverse):
    """QKV projection with the rotary embedding applied in the epilogue, against the fp32 restatement
    (bias first, then the rotation of the first heads_rot heads; the remaining columns untouched)."""
    from cogito_b200.ops.gemm import gemm, gemm_reference
    from cogito_b200.ops.misc import rope_tables
    torch.manual_seed(3)
    M, K, N = 3 * T, 200, heads_all * D
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    cos, sin = rope_tables(T + 7, D, 10000.0, DEV)
    spec = (cos, sin, heads_rot * D, D, T, 5, inverse)
    out = gemm(a, w, bias=bias, rope=spec)
    ref = gemm_reference(a, w, bias=bias, rope=spec, out_dtype=torch.float32)
    assert relerr(out, ref) < 1e-2
    # the columns behind the rotated heads are the plain projection
    plain = gemm(a, w, bias=bias)
    assert torch.equal(out[:, heads_rot * D:], plain[:, heads_rot * D:])


def test_gemm_simt_fallback_unaligned():
    from cogito_b200.ops.gemm import gemm, gemm_reference
    torch.manual_seed(0)
    a = torch.randn(77, 50, device=DEV, dtype=torch.bfloat16)   # K = 50: leading dim not a multiple of 8
    b = torch.randn(10, 50, device=DEV, dtype=torch.bfloat16)
    assert relerr(gemm(a, b), gemm_reference(a, b, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("act", [None, "gelu", "relu", "silu"])
def test_gemm_epilogues(act):
    from cogito_b200.ops.gemm import gemm, gemm_reference
    torch.manual_seed(1)
    M, N, K = 512, 384, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    aux = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, act=act, residual=res, aux_out=aux)
    ref, raux = gemm_reference(a, b, bias=bias, act=act, residual=res, want_aux=True, out_dtype=torch.float32)
    assert relerr(out, ref) < 1e-2 and relerr(aux, raux) < 1e-2
    if act:
        auxin = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
        out = gemm(a, b, aux_in=auxin, dact=act)
        ref = gemm_reference(a, b, aux_in=auxin, dact=act, out_dtype=torch.float32)
        assert relerr(out, ref) < 1e-2


def test_gemm_accumulate_fp32_and_batched():
    from cogito_b200.ops.gemm import gemm, gemm_reference
    torch.manual_seed(2)
    a = torch.randn(300, 264, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(136, 264, device=DEV, dtype=torch.bfloat16)
    acc = torch.randn(300, 136, device=DEV, dtype=torch.float32)
    ref = gemm_reference(a, b, accumulate_into=acc.clone(), out_dtype=torch.float32)
    gemm(a, b, out=acc, accumulate=True)
    assert relerr(acc, ref) < 1e-2
    a3 = torch.randn(3, 200, 64, device=DEV, dtype=torch.bfloat16)
    b3 = torch.randn(3, 136, 64, device=DEV, dtype=torch.bfloat16)
    assert relerr(gemm(a3, b3), gemm_reference(a3, b3, out_dtype=torch.float32)) < 1e-2


def test_gemm_is_deterministic():
    from cogito_b200.ops.gemm import gemm
    torch.manual_seed(3)
    a = torch.randn(1024, 512, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(768, 512, device=DEV, dtype=torch.bfloat16)
    assert torch.equal(gemm(a, b), gemm(a, b))


# ---------------------------------------------------------------- attention
CASES = [
    dict(B=1, Tq=128, Tk=128, Hq=1, Hk=1, D=64, causal=False),
    dict(B=2, Tq=512, Tk=512, Hq=4, Hk=4, D=64, causal=True),
    dict(B=2, Tq=512, Tk=512, Hq=4, Hk=4, D=128, causal=True),
    dict(B=1, Tq=300, Tk=300, Hq=2, Hk=2, D=64, causal=True),
    dict(B=1, Tq=384, Tk=640, Hq=4, Hk=2, D=64, causal=True),
    dict(B=1, Tq=1024, Tk=1024, Hq=8, Hk=2, D=128, causal=True),
    dict(B=1, Tq=1024, Tk=1024, Hq=4, Hk=1, D=64, causal=False),
    dict(B=1, Tq=1024, Tk=1024, Hq=2, Hk=2, D=64, causal=True, window=200),
    dict(B=1, Tq=700, Tk=700, Hq=2, Hk=2, D=64, causal=False, window=100),
    dict(B=1, Tq=512, Tk=512, Hq=4, Hk=4, D=64, causal=True, alibi=True),
    dict(B=1, Tq=100, Tk=900, Hq=2, Hk=2, D=128, causal=False),
]


@pytest.mark.parametrize("c", CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
def test_flash_attention_forward_backward(c):
    from cogito_b200.ops.attention import (alibi_slopes, attention_reference, flash_backward,
                                           flash_forward)
    torch.manual_seed(0)
    q = torch.randn(c["B"], c["Tq"], c["Hq"], c["D"], device=DEV, dtype=torch.bfloat16)
    k = torch.randn(c["B"], c["Tk"], c["Hk"], c["D"], device=DEV, dtype=torch.bfloat16)
    v = torch.randn(c["B"], c["Tk"], c["Hk"], c["D"], device=DEV, dtype=torch.bfloat16)
    kw = dict(causal=c["causal"], window=c.get("window", -1),
              alibi=alibi_slopes(c["Hq"], DEV) if c.get("alibi") else None)
    o, lse = flash_forward(q, k, v, **kw)
    qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ro, rlse = attention_reference(qq, kk, vv, **kw)
    fin = torch.isfinite(rlse)
    assert relerr(o, ro) < 2e-2
    assert relerr(lse[fin], rlse[fin]) < 1e-2
    do = torch.randn_like(o)
    dq, dk, dv = flash_backward(do, q, k, v, o, lse, **kw)
    gq, gk, gv = torch.autograd.grad(ro, (qq, kk, vv), do.float())
    assert relerr(dq, gq) < 3e-2 and relerr(dk, gk) < 3e-2 and relerr(dv, gv) < 3e-2


def test_packed_attention_with_rope_matches_reference():
    from cogito_b200.nn.transformer import packed_attention
    from cogito_b200.ops.misc import rope_tables
    torch.manual_seed(0)
    B, T, Hq, Hk, D = 2, 256, 4, 2, 64
    x = torch.randn(B, T, Hq + 2 * Hk, D, device=DEV, dtype=torch.bfloat16)
    cos_g, sin_g = rope_tables(T, D, 10000.0, DEV)
    cos_c, sin_c = rope_tables(T, D, 10000.0, "cpu")
    assert (cos_g.cpu() - cos_c).abs().max() < 1e-4
    xg = x.clone().requires_grad_(True)
    og = packed_attention(xg * 1.0, Hq, Hk, causal=True, scale=1 / math.sqrt(D), rope=(cos_g, sin_g))
    xc = x.float().cpu().requires_grad_(True)
    oc = packed_attention(xc * 1.0, Hq, Hk, causal=True, scale=1 / math.sqrt(D), rope=(cos_c, sin_c))
    assert relerr(og.cpu(), oc) < 2e-2
    g = torch.randn_like(og)
    og.backward(g)
    oc.backward(g.float().cpu())
    assert relerr(xg.grad.cpu(), xc.grad) < 3e-2
