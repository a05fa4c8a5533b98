"""CPU tests of the framework layer: modules, autograd, losses, optimizers, trainer.
These run without a GPU; the CPU path of every op is an fp32 restatement of the
CUDA kernel's formula."""
import math

import pytest
import torch

from cogito_b200 import nn as cnn
from cogito_b200.utils.rng import manual_seed
from cogito_b200.ops import loss as L
from cogito_b200.optim.fused import FusedAdam, FusedSGD, GradScaler, exp_lr, step_lr


def test_xor_trains_through_sequential_api():
    """Linear(2,4) -> ReLU -> Linear(4,1) -> Sigmoid, MSE, SGD lr 0.5 momentum 0.9,
    5000 full-batch epochs, seed 0: loss < 0.01 (the README example of the reference)."""
    manual_seed(0)
    model = cnn.Sequential(cnn.Linear(2, 4), cnn.ReLU(), cnn.Linear(4, 1), cnn.Sigmoid())
    opt = FusedSGD(model.parameters(), lr=0.5, momentum=0.9, master_weights=False)
    X = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]])
    Y = torch.tensor([[0.], [1.], [1.], [0.]])
    loss = None
    for _ in range(5000):
        opt.zero_grad()
        loss = L.mse_loss(model(X), Y)
        loss.backward()
        opt.step()
    assert float(loss) < 0.01
    pred = (model(X) > 0.5).float()
    assert torch.equal(pred, Y)


def test_linear_gradients_match_torch():
    torch.manual_seed(0)
    lin = cnn.Linear(7, 5, act="gelu")
    x = torch.randn(11, 7, requires_grad=True)
    res = torch.randn(11, 5, requires_grad=True)
    y = lin(x, residual=res)
    ref = torch.nn.functional.gelu(x @ lin.weight.T + lin.bias, approximate="tanh") + res
    assert torch.allclose(y, ref, atol=1e-5)
    g = torch.randn_like(y)
    gx, gw, gb, gr = torch.autograd.grad(y, (x, lin.weight, lin.bias, res), g)
    rx, rw, rb, rr = torch.autograd.grad(ref, (x, lin.weight, lin.bias, res), g)
    for a, b in ((gx, rx), (gw, rw), (gb, rb), (gr, rr)):
        assert torch.allclose(a, b, atol=1e-4)


def test_losses_match_definitions():
    torch.manual_seed(0)
    p, t = torch.randn(6, 3), torch.randn(6, 3)
    assert torch.allclose(L.mse_loss(p, t), torch.nn.functional.mse_loss(p, t))
    assert torch.allclose(L.l1_loss(p, t, "sum"), torch.nn.functional.l1_loss(p, t, reduction="sum"))
    assert torch.allclose(L.smooth_l1_loss(p, t), torch.nn.functional.smooth_l1_loss(p, t))
    pr, tb = torch.rand(6, 3), (torch.rand(6, 3) > 0.5).float()
    assert torch.allclose(L.bce_loss(pr, tb), torch.nn.functional.binary_cross_entropy(pr, tb), atol=1e-5)
    assert torch.allclose(L.bce_with_logits_loss(p, tb),
                          torch.nn.functional.binary_cross_entropy_with_logits(p, tb), atol=1e-6)
    tg = torch.randint(0, 3, (6,))
    assert torch.allclose(L.softmax_cross_entropy_small(p, tg), torch.nn.functional.cross_entropy(p, tg), atol=1e-5)
    logits = torch.randn(4, 9, 50, requires_grad=True)
    tgt = torch.randint(0, 50, (4, 9))
    tgt[0, 0] = -100
    loss = L.cross_entropy(logits * 1.0, tgt, grad_scale=2.0)
    loss.backward()
    ref_in = logits.detach().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in.view(-1, 50), tgt.view(-1), ignore_index=-100)
    ref.backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(logits.grad, 2.0 * ref_in.grad, atol=1e-5)


def test_adam_follows_reference_update_rule():
    """t++ first, decoupled decay p -= lr*wd*p, p -= lr * m_hat / (sqrt(v_hat) + eps)."""
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(10))
    p = w.detach().clone()
    opt = FusedAdam([w], lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1, master_weights=False)
    m = torch.zeros(10)
    v = torch.zeros(10)
    for t in range(1, 4):
        g = torch.randn(10)
        opt.zero_grad()
        w.main_grad.copy_(g)
        opt.step()
        p = p - 0.01 * 0.1 * p
        m = 0.9 * m + 0.1 * g
        v = 0.999 * v + 0.001 * g * g
        p = p - 0.01 * (m / (1 - 0.9 ** t)) / (torch.sqrt(v / (1 - 0.999 ** t)) + 1e-8)
        assert torch.allclose(w.detach(), p, atol=1e-6)


def test_sgd_momentum_and_nesterov_rule():
    w = torch.nn.Parameter(torch.ones(4))
    opt = FusedSGD([w], lr=0.1, momentum=0.9, weight_decay=0.5, nesterov=False, master_weights=False)
    g = torch.full((4,), 2.0)
    opt.zero_grad(); w.main_grad.copy_(g); opt.step()
    # g' = g + wd*p = 2.5 ; v = 2.5 ; p = 1 - 0.25
    assert torch.allclose(w.detach(), torch.full((4,), 0.75))
    opt.zero_grad(); w.main_grad.copy_(g); opt.step()
    gp = 2.0 + 0.5 * 0.75
    vel = 0.9 * 2.5 + gp
    assert torch.allclose(w.detach(), torch.full((4,), 0.75 - 0.1 * vel))


def test_loss_scaler_constants_and_skip():
    s = GradScaler("cpu", enabled=True)
    assert s.scale == 65536.0 and s.window == 2000 and s.min_scale == 1.0 and s.max_scale == 65536.0
    assert s.host_update(True) is True and s.scale == 32768.0
    for _ in range(1999):
        assert s.host_update(False) is False
    assert s.scale == 32768.0
    s.host_update(False)
    assert s.scale == 65536.0
    s.host_update(False)
    for _ in range(2100):
        s.host_update(False)
    assert s.scale == 65536.0          # capped at max
    t = GradScaler("cpu", enabled=True, init_scale=2.0)
    t.host_update(True); t.host_update(True)
    assert t.scale == 1.0              # floor


def test_lr_schedules():
    w = torch.nn.Parameter(torch.ones(2))
    opt = FusedSGD([w], lr=1.0, master_weights=False)
    for step in range(0, 21):
        step_lr(opt, step, 10, 0.5)
    assert opt.lr == 0.25
    exp_lr(opt, 1.0, 0.9, 3)
    assert abs(opt.lr - 0.729) < 1e-9


def test_transformer_block_variants_run_and_backprop():
    torch.manual_seed(0)
    for kw in [dict(), dict(rms_norm=True, swiglu=True, bias=False, rope=True, num_kv_heads=2),
               dict(alibi=True, window=8), dict(pre_norm=False)]:
        cfg = cnn.TransformerConfig(hidden_size=32, num_heads=4, intermediate_size=64, max_seq_len=16, **kw)
        blk = cnn.TransformerBlock(cfg)
        x = torch.randn(2, 16, 32, requires_grad=True)
        y = blk(x)
        assert y.shape == x.shape and torch.isfinite(y).all()
        y.sum().backward()
        assert x.grad is not None and torch.isfinite(x.grad).all()
        for p in blk.parameters():
            assert p.grad is not None, kw


def test_attention_block_matches_torch_sdpa():
    torch.manual_seed(0)
    cfg = cnn.TransformerConfig(hidden_size=32, num_heads=4, intermediate_size=64, max_seq_len=16)
    attn = cnn.SelfAttention(cfg)
    h = torch.randn(2, 16, 32)
    out = attn(h)
    qkv = (h @ attn.qkv.weight.T + attn.qkv.bias).view(2, 16, 12, 8)
    q, k, v = (t.transpose(1, 2) for t in (qkv[:, :, :4], qkv[:, :, 4:8], qkv[:, :, 8:]))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    ref = ref.transpose(1, 2).reshape(2, 16, 32) @ attn.proj.weight.T + attn.proj.bias
    assert torch.allclose(out, ref, atol=1e-4)


def test_gpt2_trains_on_cpu_and_trainer_accumulates_micro_batches():
    from cogito_b200.models.gpt2 import GPT2, GPT2Config
    from cogito_b200.train import Trainer
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=64, n_layer=2, d_model=32, n_head=2, d_ff=64, max_seq_len=16)
    ids = torch.randint(0, 64, (4, 16))
    tg = torch.randint(0, 64, (4, 16))
    m1, m2 = GPT2(cfg), GPT2(cfg)
    m2.load_state_dict(m1.state_dict())
    t1 = Trainer(m1, FusedAdam(m1.parameters(), lr=1e-2), micro_batch=4)
    t2 = Trainer(m2, FusedAdam(m2.parameters(), lr=1e-2), micro_batch=2)
    l1 = [float(t1.step(ids, tg)) for _ in range(8)]
    l2 = [float(t2.step(ids, tg)) for _ in range(8)]
    assert l1[-1] < l1[0] - 0.5
    assert all(abs(a - b) < 1e-3 for a, b in zip(l1, l2))      # micro-batching is exact


def test_block_recompute_gives_the_same_loss_and_gradients():
    import torch
    from cogito_b200.models.gpt2 import GPT2, GPT2Config
    from cogito_b200.utils.rng import manual_seed
    g = torch.Generator().manual_seed(3)
    ids, tg = torch.randint(0, 64, (2, 16), generator=g), torch.randint(0, 64, (2, 16), generator=g)
    grads = []
    for rc in (False, True):
        manual_seed(0)
        m = GPT2(GPT2Config(vocab_size=64, n_layer=2, d_model=32, n_head=2, d_ff=64, max_seq_len=16, recompute=rc))
        loss = m(ids, tg)
        loss.backward()
        grads.append((float(loss), [p.grad.clone() for p in m.parameters()]))
    assert abs(grads[0][0] - grads[1][0]) < 1e-6
    for a, b in zip(grads[0][1], grads[1][1]):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)


def test_softmax_dropout_residual_matches_its_unfused_chain():
    import torch
    from cogito_b200.ops.misc import softmax_dropout_residual
    torch.manual_seed(0)
    x = torch.randn(5, 7, 33, requires_grad=True)
    mul = (torch.rand(5, 7, 33) > 0.2).float() / 0.8
    res = torch.randn(5, 7, 33, requires_grad=True)
    out = softmax_dropout_residual(x, res, mul=mul)
    ref = torch.softmax(x, -1) * mul + res
    assert torch.allclose(out, ref, atol=1e-6)
    g = torch.randn_like(out)
    gx, gr = torch.autograd.grad(out, (x, res), g)
    rx, rr = torch.autograd.grad(ref, (x, res), g)
    assert torch.allclose(gx, rx, atol=1e-6) and torch.allclose(gr, rr)
    # generated mask: every kept element is softmax / (1 - p), the rest is the residual alone
    y = softmax_dropout_residual(x.detach(), None, p=0.25, seed=11)
    s = torch.softmax(x.detach(), -1)
    kept = y != 0
    assert torch.allclose(y[kept], (s / 0.75)[kept], atol=1e-6) and 0.6 < kept.float().mean() < 0.9
    assert torch.equal(softmax_dropout_residual(x.detach(), None, p=0.25, training=False), s)
