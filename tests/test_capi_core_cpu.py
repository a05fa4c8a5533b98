"""Host runtime (libcogito.so): tensors, tape autograd, layers, losses, optimizers, data,
checkpoints, profiler, bf16.  Oracles are numpy / PyTorch fp32 implementations of the same op."""
import ctypes
import shutil
import struct
import subprocess
from ctypes import POINTER, byref, c_char_p, c_float, c_int

import numpy as np
import pytest
import torch
import torch.nn.functional as Fn

from capi_defs import (FP, IP, L, ROOT, T, TensorP, TransformerConfig, borrowed, cg, grad_of)

rng = np.random.default_rng(0)


def test_tensor_ops_and_tape_gradients_match_torch():
    a_np, b_np = rng.standard_normal((3, 4), dtype=np.float32), rng.standard_normal((4, 5), dtype=np.float32)
    c_np = rng.standard_normal((5,), dtype=np.float32)
    a, b, c = T(a_np, True), T(b_np, True), T(c_np, True)
    y = ((a @ b) + c) * ((a @ b) + c)
    loss = y.mean()
    loss.backward()
    ta, tb, tc = (torch.tensor(x, requires_grad=True) for x in (a_np, b_np, c_np))
    tl = ((ta @ tb + tc) ** 2).mean()
    tl.backward()
    assert np.allclose(loss.numpy()[0], tl.item(), rtol=1e-5)
    for mine, ref in ((a, ta), (b, tb), (c, tc)):
        assert np.allclose(mine.grad, ref.grad.numpy(), rtol=1e-4, atol=1e-5)
    assert cg.infer_matmul_shape((7, 1, 3, 4), (2, 4, 5)) == (7, 2, 3, 5)
    assert cg.infer_matmul_shape(("B", 3, 4), (4, "N")) == ("B", 3, "N")
    with pytest.raises(ValueError):
        cg.infer_matmul_shape((3, 4), (5, 6))


@pytest.mark.parametrize("M,K,N", [(1, 7, 5), (3, 33, 17), (4, 8, 8), (7, 65, 31), (37, 129, 70)])
def test_host_gemm_every_operand_layout_on_ragged_sizes(M, K, N):
    """Products as the layers issue them: x W^T (forward), G W (input gradient), G^T x (weight gradient) and the
    plain a b with its two gradients, for row counts around the kernel's block of four and odd widths."""
    lib = L()
    x_np = rng.standard_normal((M, K), dtype=np.float32)
    x_np[:, ::3] = 0.0                                                # zero activations are skipped, not mis-added
    g_np = rng.standard_normal((M, N), dtype=np.float32)
    lin = lib.cg_linear_new(K, N, True)
    model = _seq(lin)
    w_np = borrowed(lin.contents.weights)
    x = T(x_np, True)
    out = lib.cg_sequential_forward(model, x._ptr)
    prod = cg.Tensor.from_ptr(out) * T(g_np)
    loss = prod.sum()
    loss.backward()
    tx, tw = torch.tensor(x_np, requires_grad=True), torch.tensor(w_np, requires_grad=True)
    tb = torch.tensor(borrowed(lin.contents.bias))
    ty = (tx @ tw if tuple(w_np.shape) == (K, N) else tx @ tw.T) + tb
    (ty * torch.tensor(g_np)).sum().backward()
    assert np.allclose(borrowed(out), ty.detach().numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(x.grad, tx.grad.numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(grad_of(lin.contents.weights), tw.grad.numpy(), rtol=1e-4, atol=1e-4)
    del prod, loss
    lib.cg_sequential_free(model)
    # a b and a b^T-shaped operands through the tape
    b_np = rng.standard_normal((K, N), dtype=np.float32)
    a, b = T(x_np, True), T(b_np, True)
    l2 = ((a @ b) * T(g_np)).sum()
    l2.backward()
    ta, tb2 = torch.tensor(x_np, requires_grad=True), torch.tensor(b_np, requires_grad=True)
    ((ta @ tb2) * torch.tensor(g_np)).sum().backward()
    assert np.allclose(a.grad, ta.grad.numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(b.grad, tb2.grad.numpy(), rtol=1e-4, atol=1e-4)


def test_batched_matmul_cat_stack_arena():
    lib = L()
    a, b = rng.standard_normal((2, 3, 4), dtype=np.float32), rng.standard_normal((2, 4, 5), dtype=np.float32)
    out = cg.Tensor((2, 3, 5))
    ta, tb = T(a), T(b)
    lib.cg_tensor_matmul(ta._ptr, tb._ptr, out._ptr)
    assert np.allclose(out.numpy(), a @ b, atol=1e-5)
    ts = [T(rng.standard_normal((2, 3), dtype=np.float32)) for _ in range(3)]
    arr = (TensorP * 3)(*[t._ptr for t in ts])
    cat = cg.Tensor.from_ptr(lib.cg_tensor_cat(arr, 3, 1))
    assert np.allclose(cat.numpy(), np.concatenate([t.numpy() for t in ts], axis=1))
    st = cg.Tensor.from_ptr(lib.cg_tensor_stack(arr, 3))
    assert st.shape == (3, 2, 3)
    arena = lib.cg_arena_new(4096)
    shape = (c_int * 2)(8, 8)
    t = lib.cg_tensor_zeros_arena(arena, shape, 2, True)
    assert t.contents.size == 64 and lib.cg_arena_total_used(arena) >= 64 * 4 * 2
    lib.cg_arena_clear(arena)
    assert lib.cg_arena_total_used(arena) == 0
    lib.cg_arena_free(arena)


def _seq(*layers):
    lib = L()
    s = lib.cg_sequential_new()
    for l in layers:
        lib.cg_sequential_add(s, l)
    return s


def _set(ptr, arr):
    c = ptr.contents
    np.ctypeslib.as_array(c.data, shape=(c.size,))[:] = np.asarray(arr, np.float32).reshape(-1)


def test_xor_converges_through_cg_backward():
    lib = L()
    lib.cg_manual_seed(0)
    model = _seq(lib.cg_linear_new(2, 4, True), lib.cg_relu_new(), lib.cg_linear_new(4, 1, True), lib.cg_sigmoid_new())
    opt = lib.cg_sgd_new_for_sequential(model, 0.5, 0.9, 0.0, False)
    x, y = T([[0, 0], [0, 1], [1, 0], [1, 1]]), T([[0], [1], [1], [0]])
    live0 = lib.cg_tensor_live_count()
    for _ in range(5000):
        lib.cg_optimizer_zero_grad(opt)
        pred = lib.cg_sequential_forward(model, x._ptr)
        loss = lib.cg_mse_loss(pred, y._ptr, 1)
        lib.cg_backward(loss)
        lib.cg_optimizer_step(opt)
        value = loss.contents.data[0]
        lib.cg_tensor_release(loss)
        lib.cg_tensor_release(pred)          # the caller's reference to the model's output (the last layer keeps its own)
    assert value < 0.01
    assert lib.cg_tensor_live_count() <= live0 + 16          # no per-step leak
    lib.cg_optimizer_free(opt)
    lib.cg_sequential_free(model)


def test_xor_example_compiles_as_c11_and_converges(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc:
        pytest.skip("no C compiler")
    exe = tmp_path / "xor"
    subprocess.check_call([cc, "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "examples" / "xor.c"),
                           "-L", str(ROOT / "cogito_b200" / "lib"), "-lcogito", "-lm", "-o", str(exe)])
    r = subprocess.run([str(exe), "5000", "0"], env={"LD_LIBRARY_PATH": str(ROOT / "cogito_b200" / "lib")}, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout
    assert "live tensors 0" in r.stdout


def test_mnist_example_trains_with_the_library_layers_loader_and_adam(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc:
        pytest.skip("no C compiler")
    exe = tmp_path / "mnist"
    subprocess.check_call([cc, "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "examples" / "mnist.c"),
                           "-L", str(ROOT / "cogito_b200" / "lib"), "-lcogito", "-lm", "-o", str(exe)])
    r = subprocess.run([str(exe)], env={"LD_LIBRARY_PATH": str(ROOT / "cogito_b200" / "lib")}, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout              # exit code 0 = final training accuracy above 0.9
    assert "epoch 5" in r.stdout


def test_device_example_runs_in_host_mode_without_a_gpu(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc:
        pytest.skip("no C compiler")
    exe = tmp_path / "device"
    subprocess.check_call([cc, "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "examples" / "device.c"),
                           "-L", str(ROOT / "cogito_b200" / "lib"), "-lcogito", "-lm", "-o", str(exe)])
    env = {"LD_LIBRARY_PATH": str(ROOT / "cogito_b200" / "lib"), "COGITO_FORCE_HOST": "1"}
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "mode: host" in r.stdout and "matches the host computation" in r.stdout


def test_layers_match_torch_forward_and_backward():
    lib = L()
    # conv -> batchnorm -> relu -> maxpool -> flatten -> linear, loss = sum(out * w)
    x_np = rng.standard_normal((2, 3, 8, 8), dtype=np.float32)
    conv, bn, pool, flat, lin = lib.cg_conv2d_new(3, 4, 3, 1, 1, True), lib.cg_batchnorm_new(4, 1e-5, 0.1), lib.cg_maxpool2d_new(2, 2), lib.cg_flatten_new(), lib.cg_linear_new(64, 5, True)
    model = _seq(conv, bn, lib.cg_relu_new(), pool, flat, lin)
    x = T(x_np, True)
    out = lib.cg_sequential_forward(model, x._ptr)
    w_np = rng.standard_normal((2, 5), dtype=np.float32)
    prod = cg.Tensor.from_ptr(out) * T(w_np)
    loss = prod.sum()
    loss.backward()
    tx = torch.tensor(x_np, requires_grad=True)
    cw = torch.tensor(borrowed(conv.contents.weights)).view(4, 3, 3, 3).requires_grad_()
    cb = torch.tensor(borrowed(conv.contents.bias), requires_grad=True)
    lw = torch.tensor(borrowed(lin.contents.weights), requires_grad=True)
    lb = torch.tensor(borrowed(lin.contents.bias), requires_grad=True)
    g, be = torch.ones(4, requires_grad=True), torch.zeros(4, requires_grad=True)
    h = Fn.conv2d(tx, cw, cb, padding=1)
    h = Fn.batch_norm(h, None, None, g, be, training=True, eps=1e-5)
    h = Fn.max_pool2d(Fn.relu(h), 2, 2).flatten(1)
    ref = h @ lw + lb
    (ref * torch.tensor(w_np)).sum().backward()
    assert np.allclose(borrowed(out), ref.detach().numpy(), atol=1e-4)
    assert np.allclose(x.grad, tx.grad.numpy(), atol=1e-4)
    assert np.allclose(grad_of(conv.contents.weights).reshape(4, 3, 3, 3), cw.grad.numpy(), atol=1e-3)
    assert np.allclose(grad_of(lin.contents.weights), lw.grad.numpy(), atol=1e-4)
    assert np.allclose(grad_of(bn.contents.weights), g.grad.numpy(), atol=1e-3)
    del prod, loss
    lib.cg_sequential_free(model)


def test_conv2d_without_bias_has_one_parameter_and_matches_torch():
    lib = L()
    conv = lib.cg_conv2d_new(2, 3, 3, 2, 1, False)
    assert not conv.contents.bias and conv.contents.num_params(conv) == 1
    x_np = rng.standard_normal((2, 2, 7, 7), dtype=np.float32)
    x = T(x_np, True)
    model = _seq(conv)
    out = lib.cg_sequential_forward(model, x._ptr)
    y = cg.Tensor.from_ptr(out)
    loss = (y * y).sum()
    loss.backward()
    tx = torch.tensor(x_np, requires_grad=True)
    tw = torch.tensor(borrowed(conv.contents.weights)).view(3, 2, 3, 3).requires_grad_()
    ty = Fn.conv2d(tx, tw, None, stride=2, padding=1)
    (ty * ty).sum().backward()
    assert np.allclose(borrowed(out), ty.detach().numpy(), atol=1e-4)
    assert np.allclose(x.grad, tx.grad.numpy(), atol=1e-3)
    assert np.allclose(grad_of(conv.contents.weights).reshape(3, 2, 3, 3), tw.grad.numpy(), atol=1e-3)
    del y, loss
    lib.cg_sequential_free(model)


def test_rmsnorm_swiglu_softmax_dropout():
    lib = L()
    x_np = rng.standard_normal((4, 8), dtype=np.float32)
    x = T(x_np, True)
    rn, sw, sm = lib.cg_rmsnorm_new(8, 1e-6), lib.cg_swiglu_new(), lib.cg_softmax_new()
    model = _seq(rn, sw, sm)
    out = lib.cg_sequential_forward(model, x._ptr)
    w_np = rng.standard_normal((4, 4), dtype=np.float32)
    loss = (cg.Tensor.from_ptr(out) * T(w_np)).sum()
    loss.backward()
    tx = torch.tensor(x_np, requires_grad=True)
    h = tx * torch.rsqrt(tx.pow(2).mean(-1, keepdim=True) + 1e-6)
    h = Fn.silu(h[:, :4]) * h[:, 4:]
    ref = torch.softmax(h, -1)
    (ref * torch.tensor(w_np)).sum().backward()
    assert np.allclose(borrowed(out), ref.detach().numpy(), atol=1e-5)
    assert np.allclose(x.grad, tx.grad.numpy(), atol=1e-4)
    del loss
    lib.cg_sequential_free(model)
    d = lib.cg_dropout_new(0.5)
    ones = T(np.ones((1000,), np.float32))
    y = borrowed(d.contents.forward(d, ones._ptr))
    assert set(np.unique(y)) <= {0.0, 2.0} and 0.35 < (y == 0).mean() < 0.65
    lib.cg_dropout_set_training(d, False)
    assert np.all(borrowed(d.contents.forward(d, ones._ptr)) == 1.0)
    lib.cg_layer_free(d)


def test_losses_match_torch():
    lib = L()
    p_np, t_np = rng.standard_normal((6, 5), dtype=np.float32), rng.standard_normal((6, 5), dtype=np.float32)
    onehot = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 6)]
    prob = 1 / (1 + np.exp(-p_np))
    cases = [
        (lambda a, b: lib.cg_mse_loss(a, b, 1), p_np, t_np, lambda a, b: Fn.mse_loss(a, b)),
        (lambda a, b: lib.cg_l1_loss(a, b, 2), p_np, t_np, lambda a, b: Fn.l1_loss(a, b, reduction="sum")),
        (lambda a, b: lib.cg_smooth_l1_loss(a, b, 0.7, 1), p_np, t_np, lambda a, b: Fn.smooth_l1_loss(a, b, beta=0.7)),
        (lambda a, b: lib.cg_bce_with_logits_loss(a, b, 1), p_np, onehot, lambda a, b: Fn.binary_cross_entropy_with_logits(a, b)),
        (lambda a, b: lib.cg_bce_loss(a, b, 1), prob, onehot, lambda a, b: Fn.binary_cross_entropy(a, b)),
        (lambda a, b: lib.cg_softmax_cross_entropy_loss(a, b, 1), p_np, onehot, lambda a, b: Fn.cross_entropy(a, b.argmax(1))),
    ]
    for mine, a_np, b_np, ref in cases:
        a = T(a_np, True)
        b = T(b_np)
        loss = cg.Tensor.from_ptr(mine(a._ptr, b._ptr))
        loss.backward()
        ta = torch.tensor(a_np, requires_grad=True)
        tl = ref(ta, torch.tensor(b_np))
        tl.backward()
        assert np.allclose(loss.numpy()[0], tl.item(), rtol=1e-4, atol=1e-6)
        assert np.allclose(a.grad, ta.grad.numpy(), rtol=1e-3, atol=1e-5)


def test_adam_sgd_schedules_loss_scaling_master_weights():
    lib = L()
    w_np, g_np = rng.standard_normal((10,), dtype=np.float32), rng.standard_normal((10,), dtype=np.float32)
    for kind in ("adam", "sgd"):
        w = T(w_np, True)
        tw = torch.tensor(w_np, requires_grad=True)
        params = (TensorP * 1)(w._ptr)
        if kind == "adam":
            opt = lib.cg_adam_new(params, 1, 0.01, 0.9, 0.999, 1e-8, 0.1)
            topt = torch.optim.AdamW([tw], lr=0.01, weight_decay=0.1)
        else:
            opt = lib.cg_sgd_new(params, 1, 0.01, 0.9, 0.01, True)
            topt = torch.optim.SGD([tw], lr=0.01, momentum=0.9, weight_decay=0.01, nesterov=True)
        for step in range(5):
            w.grad[:] = g_np * (step + 1)
            tw.grad = torch.tensor(g_np * (step + 1))
            lib.cg_optimizer_step(opt)
            topt.step()
        assert np.allclose(w.numpy(), tw.detach().numpy(), atol=1e-5), kind
        lib.cg_optimizer_step_lr(opt, 10, 10, 0.5)
        assert abs(opt.contents.learning_rate - 0.005) < 1e-9
        lib.cg_optimizer_exp_lr(opt, 0.1, 0.9)
        assert abs(opt.contents.learning_rate - 0.1 * 0.9 ** 5) < 1e-7
        lib.cg_optimizer_free(opt)
    # dynamic loss scale: overflow halves the scale and skips the step; bf16-rounded weights with fp32 masters
    w = T(w_np, True)
    opt = lib.cg_sgd_new((TensorP * 1)(w._ptr), 1, 0.1, 0.0, 0.0, False)
    lib.cg_optimizer_enable_loss_scaling(opt, 1024.0, 2.0, 2)
    lib.cg_optimizer_enable_master_weights(opt)
    before = w.numpy().copy()
    w.grad[:] = np.inf
    lib.cg_optimizer_step(opt)
    assert opt.contents.loss_scale == 512.0 and np.array_equal(w.numpy(), before)
    for _ in range(2):
        w.grad[:] = 512.0 * g_np
        lib.cg_optimizer_step(opt)
    assert opt.contents.loss_scale == 1024.0          # grew after the 2-step window
    master = borrowed(opt.contents.master_params[0])
    assert np.allclose(master, w_np.astype(np.float32) - 0.2 * g_np, atol=2e-2)
    assert np.array_equal(w.numpy(), torch.tensor(master).bfloat16().float().numpy())
    lib.cg_optimizer_free(opt)


def test_grad_check_accepts_right_and_rejects_wrong_gradient():
    lib = L()

    @ctypes.CFUNCTYPE(None, TensorP, TensorP)
    def square(inp, out):
        n = inp.contents.size
        for i in range(n):
            out.contents.data[i] = inp.contents.data[i] ** 2

    x_np = rng.standard_normal((5,), dtype=np.float32)
    x, go = T(x_np, True), T(np.ones(5, np.float32))
    x.grad[:] = 2 * x_np
    assert lib.cg_grad_check(square, x._ptr, go._ptr, 1e-3, 1e-2)
    x.grad[:] = 3 * x_np
    assert not lib.cg_grad_check(square, x._ptr, go._ptr, 1e-3, 1e-2)


def test_checkpoint_byte_layout_and_round_trip(tmp_path):
    lib = L()
    a, b = T(np.arange(6, dtype=np.float32).reshape(2, 3)), T(np.array([1.5, -2.5], np.float32))
    path = str(tmp_path / "m.cog").encode()
    names = (c_char_p * 2)(b"layer0.weight", b"layer0.bias")
    lib.cg_save_model(path, (TensorP * 2)(a._ptr, b._ptr), names, 2)
    raw = open(path, "rb").read()
    assert raw[:4] == bytes([0x31, 0x47, 0x4F, 0x43])
    magic, version, count, _pad, total = struct.unpack_from("<IIIIQ", raw, 0)
    assert (magic, version, count, total) == (0x434F4731, 1, 2, len(raw))
    e0 = raw[24:144]
    assert e0[:64].rstrip(b"\0") == b"layer0.weight"
    ndim, = struct.unpack_from("<i", e0, 64)
    shape = struct.unpack_from("<8i", e0, 68)
    dtype, = struct.unpack_from("<i", e0, 100)
    offset, size = struct.unpack_from("<QQ", e0, 104)
    assert (ndim, shape[:2], dtype, offset, size) == (2, (2, 3), 0, 24 + 240, 24)
    assert np.array_equal(np.frombuffer(raw, np.float32, 6, offset), np.arange(6, dtype=np.float32))
    e1_off, e1_size = struct.unpack_from("<QQ", raw, 144 + 104)
    assert (e1_off, e1_size) == (24 + 240 + 24, 8)
    ts, ns, n = POINTER(TensorP)(), POINTER(c_char_p)(), c_int()
    lib.cg_load_model(path, byref(ts), byref(ns), byref(n))
    assert n.value == 2 and ns[0] == b"layer0.weight" and ns[1] == b"layer0.bias"
    assert np.array_equal(borrowed(ts[0]), a.numpy()) and np.array_equal(borrowed(ts[1]), b.numpy())
    open(path, "wb").write(b"XXXX" + raw[4:])
    lib.cg_load_model(path, byref(ts), byref(ns), byref(n))
    assert n.value == 0 and lib.cg_last_error() == 6       # CG_ERROR_INVALID_FORMAT


def test_data_pipeline(tmp_path):
    lib = L()
    imgs = rng.integers(0, 256, (10, 4, 4), dtype=np.uint8)
    labs = rng.integers(0, 10, 10).astype(np.uint8)
    (tmp_path / "img").write_bytes(struct.pack(">IIII", 2051, 10, 4, 4) + imgs.tobytes())
    (tmp_path / "lab").write_bytes(struct.pack(">II", 2049, 10) + labs.tobytes())

    class Mnist(ctypes.Structure):
        _fields_ = [("images", TensorP), ("labels", TensorP), ("num_samples", c_int), ("rows", c_int), ("cols", c_int)]

    m = ctypes.cast(lib.cg_mnist_load(str(tmp_path / "img").encode(), str(tmp_path / "lab").encode()), POINTER(Mnist))
    assert m.contents.num_samples == 10
    assert np.allclose(borrowed(m.contents.images), imgs.reshape(10, 16) / 255.0)
    assert np.array_equal(borrowed(m.contents.labels), labs.astype(np.float32))
    loader = lib.cg_dataloader_new(m.contents.images, m.contents.labels, 4, True, 7)
    assert lib.cg_dataloader_num_batches(loader) == 3
    seen, bd, bl, n = [], TensorP(), TensorP(), c_int()
    sizes = []
    while lib.cg_dataloader_next(loader, byref(bd), byref(bl), byref(n)):
        sizes.append(n.value)
        seen.extend(borrowed(bl).tolist())
    assert sizes == [4, 4, 2] and sorted(seen) == sorted(labs.astype(np.float32).tolist())
    lib.cg_dataloader_free(loader)
    oh = cg.Tensor.from_ptr(lib.cg_tensor_onehot(m.contents.labels, 10))
    assert np.array_equal(oh.numpy().argmax(1), labs) and oh.numpy().sum() == 10
    assert lib.cg_compute_accuracy(oh._ptr, m.contents.labels, 10) == 1.0
    lib.cg_mnist_free(m)
    assert not lib.cg_mnist_load(b"/nonexistent", b"/nonexistent") and lib.cg_last_error() == 5


def test_profiler_and_bf16():
    lib = L()
    lib.cg_profiler_init()
    for _ in range(3):
        lib.cg_profiler_begin_layer(b"fc1")
        lib.cg_profiler_end_layer(b"fc1")
    assert lib.cg_profiler_count(b"fc1") == 3 and lib.cg_profiler_total_ms(b"fc1") >= 0.0
    lib.cg_profiler_reset()
    assert lib.cg_profiler_count(b"fc1") == 0
    xs = np.concatenate([rng.standard_normal(200).astype(np.float32) * 100, np.array([0.0, 1.0, 1.00390625, 3.3895314e38, np.inf, -np.inf], np.float32)])
    ref = torch.tensor(xs).bfloat16()
    for v, r in zip(xs, ref):
        h = lib.cg_fp32_to_bf16(float(v))
        assert h == (r.view(torch.int16).item() & 0xFFFF)
        assert lib.cg_bf16_to_fp32(h) == r.float().item()
    assert np.isnan(lib.cg_bf16_to_fp32(lib.cg_fp32_to_bf16(float("nan"))))


def test_mixed_precision_skips_on_overflow():
    lib = L()
    w = T(np.ones(4, np.float32), True)
    mp = lib.cg_mixed_precision_new((TensorP * 1)(w._ptr), 1)
    assert mp.contents.loss_scale == 65536.0
    w.grad[:] = [1.0, np.inf, 0.0, 0.0]
    assert not lib.cg_mp_backward(mp, None)
    lib.cg_mp_step(mp)
    assert mp.contents.loss_scale == 32768.0 and np.array_equal(w.numpy(), np.ones(4)) and mp.contents.num_skipped == 1
    w.grad[:] = 32768.0 * np.array([0.1, 0.2, 0.0, 0.0], np.float32)
    assert lib.cg_mp_backward(mp, None)
    mp.contents.learning_rate = 0.5
    mp.contents.max_grad_norm = 0.0
    lib.cg_mp_step(mp)
    assert np.allclose(w.numpy(), [0.95, 0.9, 1.0, 1.0], atol=1e-6)
    lib.cg_mixed_precision_free(mp)


def _finite_difference(fn, arr, idx, eps=1e-3):
    keep = arr[idx]
    arr[idx] = keep + eps
    hi = fn()
    arr[idx] = keep - eps
    lo = fn()
    arr[idx] = keep
    return (hi - lo) / (2 * eps)


@pytest.mark.parametrize("llama_style", [True, False])
def test_transformer_block_gradients(llama_style):
    lib = L()
    lib.cg_manual_seed(3)
    cfg = TransformerConfig(hidden_size=16, num_heads=4, num_kv_heads=2 if llama_style else 4, head_dim=4, intermediate_size=24,
                            norm_eps=1e-5, dropout_prob=0.0, use_bias=not llama_style, pre_norm=True, use_rms_norm=llama_style,
                            use_swiglu=llama_style)
    blk = lib.cg_transformer_block_new(cfg)
    n = blk.contents.num_params(blk)
    assert n == (9 if llama_style else 16)
    x = T(rng.standard_normal((5, 16), dtype=np.float32), True)
    w = T(rng.standard_normal((5, 16), dtype=np.float32))

    def run():
        out = lib.cg_transformer_forward(blk, x._ptr, None)
        return float((borrowed(out) * w.numpy()).sum())

    out = lib.cg_transformer_forward(blk, x._ptr, None)
    loss = (cg.Tensor.from_ptr(out) * w).sum()
    loss.backward()
    params = blk.contents.get_params(blk)
    xs = x.numpy()
    for idx in [(0, 0), (2, 5), (4, 15)]:
        assert abs(_finite_difference(run, xs, idx) - x.grad[idx]) < 2e-2 * max(1.0, abs(x.grad[idx]))
    for p in (0, 2, n - 1):
        c = params[p].contents
        data = np.ctypeslib.as_array(c.data, shape=(c.size,))
        ana = np.ctypeslib.as_array(c.grad, shape=(c.size,)).copy()
        for j in (0, c.size // 2, c.size - 1):
            assert abs(_finite_difference(run, data, j) - ana[j]) < 2e-2 * max(1.0, abs(ana[j])), (p, j)
    # causal: changing a later token must not change earlier outputs
    base = borrowed(lib.cg_transformer_forward(blk, x._ptr, None))
    xs[4] += 1.0
    moved = borrowed(lib.cg_transformer_forward(blk, x._ptr, None))
    assert np.allclose(base[:4], moved[:4], atol=1e-6) and not np.allclose(base[4], moved[4])
    del loss
    lib.cg_layer_free(blk)


def test_transformer_block_loop_in_c_keeps_the_live_tensor_count_flat(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    exe = tmp_path / "block_loop"
    lib = ROOT / "cogito_b200" / "lib"
    p = subprocess.run([cc, "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "tests" / "capi_block_loop.c"), "-L", str(lib),
                        "-lcogito", "-lm", f"-Wl,-rpath,{lib}", "-o", str(exe)], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == "live 0", (r.returncode, r.stdout, r.stderr)
