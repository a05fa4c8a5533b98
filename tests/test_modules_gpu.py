"""GPU tests of the newer modules: NVRTC JIT, conv / pool / batch norm, Llama training,
bf16 checkpoints, profiler, and the bounded-wait self-test (failure detection without a fault)."""
import ctypes

import pytest
import torch
import torch.nn.functional as Fn

from cogito_b200 import jit
from cogito_b200.io import checkpoint as ckpt
from cogito_b200.models.llama import Llama, LlamaConfig
from cogito_b200.models.mlp import MLPClassifier
from cogito_b200.nn import BatchNorm, Conv2d, MaxPool2d
from cogito_b200.ops import _lib
from cogito_b200.optim.fused import FusedAdam, GradScaler
from cogito_b200.train import Trainer
from cogito_b200.utils import rng
from cogito_b200.utils.profiler import Profiler, instrument

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_jit_kernel_matches_fp32_reference():
    f = jit.fuse(lambda x, b, s: jit.tanh(jit.gelu(x + b) * s) / (jit.sqrt(jit.exp(x) + 1.0)) - jit.relu(-x))
    x, b, s = torch.randn(1000, 384), torch.randn(384), torch.tensor([0.7])
    ref = torch.tanh(Fn.gelu(x + b, approximate="tanh") * s) / torch.sqrt(torch.exp(x) + 1.0) - torch.relu(-x)
    got = f(x.to(DEV), b.to(DEV), s.to(DEV))
    assert torch.allclose(got.cpu(), ref, atol=1e-5, rtol=1e-5)
    got16 = f(x.to(DEV).bfloat16(), b.to(DEV), s.to(DEV))
    ref16 = torch.tanh(Fn.gelu(x.bfloat16().float() + b, approximate="tanh") * s) / torch.sqrt(torch.exp(x.bfloat16().float()) + 1.0) - torch.relu(-x.bfloat16().float())
    assert got16.dtype == torch.bfloat16 and torch.allclose(got16.float().cpu(), ref16, atol=2e-2, rtol=2e-2)
    assert f.launches == 2 and len(f._kernels) == 2          # one compiled kernel per dtype signature


def test_conv_pool_batchnorm_match_torch():
    torch.manual_seed(0)
    rng.manual_seed(0)
    conv, pool, bn = Conv2d(3, 16, 3, stride=1, padding=1, device=DEV), MaxPool2d(2), BatchNorm(16, device=DEV)
    x = torch.randn(4, 3, 16, 16, device=DEV, requires_grad=True)
    y = pool(bn(conv(x)))
    w = torch.randn_like(y)
    (y * w).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    cw = conv.weight.detach().clone().view(16, 3, 3, 3).requires_grad_(True)
    cb = conv.bias.detach().clone().requires_grad_(True)
    g, be = torch.ones(16, device=DEV, requires_grad=True), torch.zeros(16, device=DEV, requires_grad=True)
    # the kernel path rounds the unfolded input and the weights to bf16: do the same in the oracle
    h = Fn.conv2d(xr.bfloat16().float(), cw.bfloat16().float(), cb.bfloat16().float(), padding=1)
    yr = Fn.max_pool2d(Fn.batch_norm(h, None, None, g, be, training=True, eps=1e-5), 2)
    (yr * w).sum().backward()
    assert (y - yr).abs().max().item() < 2e-2
    assert (x.grad - xr.grad).abs().max().item() < 0.05 * xr.grad.abs().max().item() + 1e-2
    assert (conv.weight.grad.view(16, 3, 3, 3) - cw.grad).abs().max().item() < 0.05 * cw.grad.abs().max().item() + 1e-2
    # bf16 noise in the convolution flips some arg-max choices of the pooling: compare directions
    assert Fn.cosine_similarity(bn.weight.grad, g.grad, dim=0).item() > 0.99
    # running = momentum * running + (1 - momentum) * batch, from (0, 1)
    assert torch.allclose(bn.running_mean, 0.9 * h.mean((0, 2, 3)).detach(), atol=1e-2)
    assert torch.allclose(bn.running_var, 0.1 + 0.9 * h.var((0, 2, 3), unbiased=False).detach(), atol=1e-2)


def test_llama_and_mlp_train_in_bf16_with_loss_scaling():
    rng.manual_seed(0)
    cfg = LlamaConfig(vocab_size=2048, n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, max_seq_len=256)
    model = Llama(cfg, device=DEV, dtype=torch.bfloat16)
    opt = FusedAdam(model.parameters(), lr=2e-3, scaler=GradScaler(DEV), max_grad_norm=1.0)
    tr = Trainer(model, opt, micro_batch=2)
    ids = torch.randint(0, 2048, (4, 256), device=DEV)
    losses = [float(tr.step(ids, ids.roll(-1, 1))) for _ in range(12)]
    assert losses[-1] < losses[0] - 0.5, losses
    mlp = MLPClassifier(784, (512, 512), 10, device=DEV, dtype=torch.bfloat16)
    o2 = FusedAdam(mlp.parameters(), lr=1e-3, scaler=GradScaler(DEV))
    t2 = Trainer(mlp, o2)
    x, y = torch.rand(256, 784, device=DEV), torch.randint(0, 10, (256,), device=DEV)
    l2 = [float(t2.step(x, y)) for _ in range(30)]
    assert l2[-1] < 0.5 * l2[0], l2
    _lib.assert_device_ok()


def test_bf16_checkpoint_round_trip_and_profiler(tmp_path):
    rng.manual_seed(1)
    cfg = LlamaConfig(vocab_size=512, n_layer=1, d_model=128, n_head=2, n_kv_head=1, d_ff=256, max_seq_len=64)
    a, b = Llama(cfg, device=DEV, dtype=torch.bfloat16), Llama(cfg, device=DEV, dtype=torch.bfloat16)
    path = str(tmp_path / "m.cog")
    ckpt.save_model(path, a)
    ckpt.load_model(path, b)
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.equal(pa, pb)
    prof = Profiler()
    instrument(a, prof, depth=2)
    ids = torch.randint(0, 512, (2, 64), device=DEV)
    a(ids)
    prof.step_end()
    assert prof.total_ms("blocks.0") > 0 and prof.stats["blocks.0"][2] > 0      # device time and kernel launches per range


def test_bounded_wait_times_out_with_a_status_and_the_context_survives():
    L = _lib.lib()
    L.cgk_selftest_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
    _lib.read_status()                                       # clear
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)     # nothing ever sets it
    reached = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.check(L.cgk_selftest_bounded_wait(flag.data_ptr(), 1, 200_000_000, reached.data_ptr(), _lib.stream_ptr()))
    t1.record()
    code, where, block, aux = _lib.read_status()
    assert (code, where, aux) == (2, 900, 1) and int(reached) == 0
    assert 150 < t0.elapsed_time(t1) < 1500                  # gave up after about the 0.2 s limit
    # a flag that is already set passes at once and leaves the status clean
    flag.fill_(3)
    _lib.check(L.cgk_selftest_bounded_wait(flag.data_ptr(), 2, 200_000_000, reached.data_ptr(), _lib.stream_ptr()))
    assert _lib.read_status()[0] == 0 and int(reached) == 1
    assert torch.ones(4, device=DEV).sum().item() == 4       # the context is intact


def test_attention_with_rotary_epilogue_matches_the_unfused_path():
    """SelfAttention with RoPE: on the GPU the QKV GEMM rotates q and k in its epilogue; the CPU path
    rotates the projection buffer in a pass of its own.  Same outputs and gradients."""
    import copy
    from cogito_b200.nn.transformer import SelfAttention, TransformerConfig
    from cogito_b200.utils.rng import manual_seed
    manual_seed(0)
    for D, Hq, Hk in ((64, 4, 2), (128, 2, 1)):
        cfg = TransformerConfig(hidden_size=Hq * D, num_heads=Hq, num_kv_heads=Hk, head_dim=D, bias=False, rope=True, max_seq_len=96)
        cpu = SelfAttention(cfg)
        gpu = copy.deepcopy(cpu).to("cuda", torch.bfloat16)
        x = torch.randn(2, 96, Hq * D)
        xc = x.clone().requires_grad_(True)
        xg = x.to("cuda", torch.bfloat16).requires_grad_(True)
        yc, yg = cpu(xc), gpu(xg)
        g = torch.randn_like(yc)
        yc.backward(g)
        yg.backward(g.to("cuda", torch.bfloat16))
        rel = lambda a, b: float((a.float().cpu() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))
        assert rel(yg, yc) < 3e-2
        assert rel(xg.grad, xc.grad) < 4e-2
        assert rel(gpu.qkv.weight.grad, cpu.qkv.weight.grad) < 4e-2
