"""Norm, loss, elementwise, reduction, embedding and optimizer kernels against
PyTorch fp32 on a B200."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def relerr(x, ref):
    x, ref = x.float().cpu(), ref.float().cpu()
    return ((x - ref).abs().max() / (ref.abs().max() + 1e-6)).item()


@pytest.mark.parametrize("rows,D", [(64, 768), (33, 128), (1000, 4096), (7, 8)])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("with_res", [False, True])
def test_norm_forward_backward(rows, D, rms, with_res):
    from cogito_b200.ops import norm as N
    torch.manual_seed(0)
    x = torch.randn(rows, D, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(rows, D, device=DEV, dtype=torch.bfloat16) if with_res else None
    g = (torch.randn(D, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    b = None if rms else (torch.randn(D, device=DEV) * 0.1).to(torch.bfloat16)
    xs = [t.clone().requires_grad_(True) for t in (x, g)] + ([b.clone().requires_grad_(True)] if b is not None else [])
    rg = r.clone().requires_grad_(True) if with_res else None
    out = N.rms_norm(xs[0], xs[1], 1e-5, rg) if rms else N.layer_norm(xs[0], xs[1], xs[2], 1e-5, rg)
    y, s = out if with_res else (out, None)
    # fp32 oracle
    xf = x.float().requires_grad_(True)
    rf = r.float().requires_grad_(True) if with_res else None
    gf = g.float().requires_grad_(True)
    bf = b.float().requires_grad_(True) if b is not None else None
    sf = xf + rf if with_res else xf
    if with_res:
        sf = sf.detach().to(torch.bfloat16).float() + (sf - sf.detach())   # the kernel rounds the sum to bf16
    if rms:
        yf = sf * torch.rsqrt((sf * sf).mean(-1, keepdim=True) + 1e-5) * gf
    else:
        yf = torch.nn.functional.layer_norm(sf, (D,), gf, bf, 1e-5)
    assert relerr(y, yf) < 2e-2
    dy = torch.randn_like(y)
    ds = torch.randn_like(y) if with_res else None
    if with_res:
        torch.autograd.backward([y, s], [dy, ds])
        torch.autograd.backward([yf, sf], [dy.float(), ds.float()])
    else:
        y.backward(dy)
        yf.backward(dy.float())
    assert relerr(xs[0].grad, xf.grad) < 3e-2
    assert relerr(xs[1].grad, gf.grad) < 3e-2
    if b is not None:
        assert relerr(xs[2].grad, bf.grad) < 3e-2
    if with_res:
        assert relerr(rg.grad, rf.grad) < 3e-2


@pytest.mark.parametrize("R,V", [(64, 50304), (33, 32000), (5, 1000), (16, 10)])
def test_fused_cross_entropy(R, V):
    from cogito_b200.ops.loss import cross_entropy
    torch.manual_seed(0)
    logits = (torch.randn(R, V, device=DEV) * 2).to(torch.bfloat16)
    tg = torch.randint(0, V, (R,), device=DEV)
    tg[0] = -100
    ref_in = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, tg, ignore_index=-100)
    ref.backward()
    x = logits.clone().requires_grad_(True)
    y = x * 1.0
    loss = cross_entropy(y, tg, grad_scale=4.0)
    loss.backward()
    assert abs(float(loss) - float(ref)) < 2e-2 * max(1.0, abs(float(ref)))
    assert relerr(x.grad, ref_in.grad * 4.0) < 3e-2
    # device-resident scale
    x2 = logits.clone().requires_grad_(True)
    loss2 = cross_entropy(x2 * 1.0, tg, grad_scale=torch.tensor([4.0], device=DEV))
    loss2.backward()
    assert relerr(x2.grad, ref_in.grad * 4.0) < 3e-2


def test_ce_stats_and_backward_split():
    import ctypes
    from cogito_b200.ops import _lib
    torch.manual_seed(0)
    R, V = 40, 4096
    logits = torch.randn(R, V, device=DEV).to(torch.bfloat16)
    tg = torch.randint(0, V, (R,), device=DEV)
    L = _lib.lib()
    halves = []
    for s in range(2):
        sh = logits[:, s * V // 2:(s + 1) * V // 2].contiguous()
        mx, sm, tl = (torch.empty(R, device=DEV) for _ in range(3))
        _lib.check(L.cgk_ce_stats(sh.data_ptr(), tg.data_ptr(), s * V // 2, mx.data_ptr(), sm.data_ptr(),
                                  tl.data_ptr(), R, V // 2, V // 2, _lib.stream_ptr()))
        halves.append((sh, mx, sm, tl))
    gmax = torch.maximum(halves[0][1], halves[1][1])
    gsum = sum(h[2] * torch.exp(h[1] - gmax) for h in halves)
    lse = gmax + torch.log(gsum)
    tgt = halves[0][3] + halves[1][3]
    ref = torch.nn.functional.cross_entropy(logits.float(), tg, reduction="none")
    assert relerr(lse - tgt, ref) < 1e-2
    probs = torch.softmax(logits.float(), -1)
    probs[torch.arange(R), tg] -= 1
    for s, (sh, *_rest) in enumerate(halves):
        d = torch.empty_like(sh)
        _lib.check(L.cgk_ce_backward(sh.data_ptr(), tg.data_ptr(), s * V // 2, lse.data_ptr(), d.data_ptr(), R,
                                     V // 2, V // 2, 1.0, None, -100, _lib.stream_ptr()))
        assert relerr(d, probs[:, s * V // 2:(s + 1) * V // 2]) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise_and_broadcast(dtype):
    from cogito_b200.ops import functional as F
    torch.manual_seed(0)
    a = torch.randn(5, 1, 33, device=DEV).to(dtype)
    b = torch.randn(1, 7, 33, device=DEV).to(dtype)
    for op, fn in [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div)]:
        bb = b + 3 if op == "div" else b
        assert relerr(F.binary(op, a, bb), fn(a.float(), bb.float())) < 2e-2
    big = torch.randn(1 << 16, device=DEV).to(dtype)
    assert relerr(F.binary("add", big, big), big.float() * 2) < 1e-2
    x = torch.rand(1000, device=DEV).to(dtype) + 0.5
    for op, fn in [("exp", torch.exp), ("log", torch.log), ("sqrt", torch.sqrt), ("tanh", torch.tanh),
                   ("sigmoid", torch.sigmoid), ("relu", torch.relu), ("rsqrt", torch.rsqrt),
                   ("gelu", lambda t: torch.nn.functional.gelu(t, approximate="tanh")),
                   ("silu", torch.nn.functional.silu)]:
        assert relerr(F.unary(op, x), fn(x.float())) < 2e-2, op
        xr = x.float().clone().detach().requires_grad_(True)
        fn(xr).sum().backward()
        dy = torch.ones_like(x)
        assert relerr(F.unary_backward(op, x, dy), xr.grad) < 3e-2, op
    assert relerr(F.unary("pow", x, 3.0), x.float() ** 3) < 2e-2


def test_large_elementwise_beyond_16M_elements():
    """The reference's grid cap (65535 blocks, no stride loop) breaks above 16.7 M elements."""
    from cogito_b200.ops import functional as F
    n = (1 << 24) + 12345
    a = torch.ones(n, device=DEV)
    out = F.binary("add", a, a)
    assert float(out.min()) == 2.0 and float(out[-1]) == 2.0


def test_reductions():
    from cogito_b200.ops import functional as F
    torch.manual_seed(0)
    x = torch.randn(6, 50, 9, device=DEV)
    for op, fn in [("sum", torch.sum), ("mean", torch.mean)]:
        assert relerr(F.reduce(op, x), fn(x).reshape(1)) < 1e-4
        for d in range(3):
            assert relerr(F.reduce(op, x, d), fn(x, d)) < 1e-4
    assert relerr(F.reduce("max", x, 1), x.max(1).values) == 0
    assert relerr(F.reduce("min", x), x.min().reshape(1)) == 0
    m = torch.randn(777, 100, device=DEV).to(torch.bfloat16)
    assert relerr(F.colsum(m), m.float().sum(0)) < 1e-3


def test_embedding_swiglu_dropout():
    from cogito_b200.ops import misc as M
    torch.manual_seed(0)
    V, D, B, T = 100, 64, 3, 17
    wte = torch.randn(V, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    wpe = torch.randn(32, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    ids = torch.randint(0, V, (B, T), device=DEV)
    out = M.embedding(ids, wte, wpe)
    ref = wte.float()[ids] + wpe.float()[:T][None]
    assert relerr(out, ref) < 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    rw = torch.zeros(V, D, device=DEV).index_add_(0, ids.reshape(-1), g.float().reshape(-1, D))
    assert relerr(wte.grad, rw) < 2e-2
    assert relerr(wpe.grad[:T], g.float().sum(0)) < 2e-2
    x = torch.randn(9, 2 * 40, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = M.swiglu(x)
    xf = x.detach().float().requires_grad_(True)
    yf = torch.nn.functional.silu(xf[:, :40]) * xf[:, 40:]
    assert relerr(y, yf) < 2e-2
    gy = torch.randn_like(y)
    y.backward(gy)
    yf.backward(gy.float())
    assert relerr(x.grad, xf.grad) < 3e-2
    z = torch.ones(100000, device=DEV)
    d = M.dropout(z, 0.25, True, seed=7)
    kept = (d != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.01 and abs(float(d.max()) - 1 / 0.75) < 1e-5
    assert torch.equal(d, M.dropout(z, 0.25, True, seed=7))


def test_fused_adam_and_scaler_match_cpu_rule():
    from cogito_b200.optim.fused import FusedAdam, GradScaler
    torch.manual_seed(0)
    w_g = torch.nn.Parameter(torch.randn(300, 17, device=DEV).to(torch.bfloat16))
    w_c = torch.nn.Parameter(w_g.detach().float().cpu().clone())
    og = FusedAdam([w_g], lr=1e-2, weight_decay=0.1, scaler=GradScaler(DEV, enabled=True, init_scale=1024.0))
    oc = FusedAdam([w_c], lr=1e-2, weight_decay=0.1, scaler=GradScaler("cpu", enabled=True, init_scale=1024.0))
    for step in range(4):
        g = torch.randn(300, 17)
        if step == 2:
            g[0, 0] = float("inf")          # overflow: both must skip and halve the scale
        og.zero_grad(); oc.zero_grad()
        w_g.main_grad.copy_((g * og.scaler.sync()["scale"]).to(DEV))
        w_c.main_grad.copy_(g * oc.scaler.scale)
        og.step(); oc.step()
    sg, sc = og.scaler.sync(), oc.scaler.sync()
    assert sg["scale"] == sc["scale"] == 512.0 and sg["skipped"] == sc["skipped"] == 1 and sg["step"] == sc["step"] == 3
    assert relerr(og.master, oc.fp.flat) < 1e-5
    assert relerr(w_g, w_c) < 1e-2


def test_fused_sgd_nesterov_matches_torch():
    from cogito_b200.optim.fused import FusedSGD
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(1000, device=DEV))
    wt = torch.nn.Parameter(w.detach().clone())
    o = FusedSGD([w], lr=0.1, momentum=0.9, weight_decay=0.01, nesterov=True, master_weights=False)
    ot = torch.optim.SGD([wt], lr=0.1, momentum=0.9, weight_decay=0.01, nesterov=True)
    for _ in range(5):
        g = torch.randn(1000, device=DEV)
        o.zero_grad(); w.main_grad.copy_(g); o.step()
        wt.grad = g.clone(); ot.step()
    assert relerr(w, wt) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_dropout_residual_kernel(dtype):
    """One row kernel for softmax -> multiply -> add, against the three separate steps."""
    from cogito_b200.ops.misc import _dropout_apply, softmax_dropout_residual
    torch.manual_seed(0)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    x = torch.randn(37, 4, 1000, device="cuda").to(dtype).requires_grad_(True)
    res = torch.randn(37, 4, 1000, device="cuda").to(dtype).requires_grad_(True)
    mul = ((torch.rand(37, 4, 1000, device="cuda") > 0.3).float() / 0.7).to(dtype)
    out = softmax_dropout_residual(x, res, mul=mul)
    ref = torch.softmax(x.float(), -1) * mul.float() + res.float()
    assert (out.float() - ref).abs().max() < tol
    g = torch.randn_like(out)
    gx, gr = torch.autograd.grad(out, (x, res), g)
    rx, rr = torch.autograd.grad(ref, (x, res), g.float())
    assert (gx.float() - rx.float()).abs().max() < tol * max(1.0, float(rx.abs().max())) and torch.equal(gr, g)
    # generated mask = the mask of the stand-alone dropout kernel for the same seed
    y = softmax_dropout_residual(x.detach(), res.detach(), p=0.2, seed=77)
    s = torch.softmax(x.detach().float(), -1)
    sep = _dropout_apply(s, 0.2, 77) + res.detach().float()
    assert (y.float() - sep).abs().max() < tol
    x2 = x.detach().clone().requires_grad_(True)
    y2 = softmax_dropout_residual(x2, None, p=0.2, seed=77)
    (g2,) = torch.autograd.grad(y2, x2, g)
    xs = x.detach().float().requires_grad_(True)
    keep = _dropout_apply(torch.ones_like(xs), 0.2, 77)          # the mask itself, scaled by 1 / (1 - p)
    (r2,) = torch.autograd.grad(torch.softmax(xs, -1) * keep, xs, g.float())
    assert (g2.float() - r2).abs().max() < tol * max(1.0, float(r2.abs().max()))
