"""Host runtime (libcogito.so): quantisation, KV cache, attention, samplers and speculative
decoding, pipeline schedules and executor, memory, symbolic shapes, JIT and fusion."""
import ctypes
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int64, c_void_p

import numpy as np
import pytest
import torch

from capi_defs import (FP, IP, L, LogitsFn, T, TensorP, borrowed, cg, grad_of, take_string)

rng = np.random.default_rng(1)


# ------------------------------------------------------------------ quantisation
def test_int4_packing_is_bit_exact_and_matmul_matches_dequant():
    lib = L()
    w_np = rng.standard_normal((16, 32), dtype=np.float32)
    w_np[0, 0], w_np[0, 1] = -3.0, 7.0
    w_np[0, 2:32] = np.clip(w_np[0, 2:32], -6.9, 6.9)
    w = T(w_np)
    q = lib.cg_quantize_int4(w._ptr, 32)
    qc = q.contents
    assert (qc.num_groups, qc.group_size, qc.size) == (16, 32, 512)
    assert abs(qc.scales[0] - 1.0) < 1e-7 and qc.data[0] == 0x7D          # even index in the low nibble
    flat = w_np.reshape(-1)
    packed = np.ctypeslib.as_array(qc.data, shape=(256,))
    for g in range(16):
        seg = flat[g * 32:(g + 1) * 32]
        scale = np.float32(np.abs(seg).max() / np.float32(7.0))
        assert np.float32(qc.scales[g]) == scale
        ref = np.clip(np.sign(seg / scale) * np.floor(np.abs(seg / scale) + 0.5), -8, 7).astype(np.int32)
        lo, hi = packed[g * 16:(g + 1) * 16] & 0xF, packed[g * 16:(g + 1) * 16] >> 4
        got = np.stack([lo, hi], 1).reshape(-1).astype(np.int32)
        got = np.where(got >= 8, got - 16, got)
        assert np.array_equal(got, ref)
    deq = cg.Tensor.from_ptr(lib.cg_dequantize(q))
    assert np.abs(deq.numpy() - w_np).max() <= np.abs(w_np).max() / 14 + 1e-6
    x_np = rng.standard_normal((3, 16), dtype=np.float32)
    x, out, gv = T(x_np), cg.Tensor((3, 32)), cg.Tensor((32,))
    lib.cg_matmul_int4(x._ptr, q, out._ptr)
    assert np.allclose(out.numpy(), x_np @ deq.numpy(), atol=1e-4)
    row = T(x_np[0])
    lib.cg_gemv_int4(row._ptr, q, gv._ptr)
    assert np.allclose(gv.numpy(), out.numpy()[0], atol=1e-5)
    lib.cg_tensor_quant_free(q)


def test_nf4_gptq_awq_reduce_the_error_they_target():
    lib = L()
    w_np = (rng.standard_normal((32, 64)) * 0.5).astype(np.float32)
    w = T(w_np)

    def deq(q):
        t = cg.Tensor.from_ptr(lib.cg_dequantize(q))
        lib.cg_tensor_quant_free(q)
        return t.numpy().copy()

    plain = deq(lib.cg_quantize_int4(w._ptr, 64))
    nf4 = deq(lib.cg_quantize_nf4(w._ptr, 64))
    assert np.mean((nf4 - w_np) ** 2) < np.mean((plain - w_np) ** 2)          # normal-float levels fit Gaussian weights
    # GPTQ minimises the output error under correlated inputs
    base = rng.standard_normal((256, 8)).astype(np.float32)
    X = (base @ rng.standard_normal((8, 64)).astype(np.float32) + 0.1 * rng.standard_normal((256, 64))).astype(np.float32)
    H = T(X.T @ X)
    gptq = deq(lib.cg_quantize_gptq(w._ptr, H._ptr, 64, 4))
    err = lambda wq: np.linalg.norm(X @ (wq - w_np).T)
    assert err(gptq) < 0.9 * err(plain)
    # AWQ protects the input channels that carry large activations
    act_np = (rng.standard_normal((128, 64)) * np.where(np.arange(64) % 8 == 0, 20.0, 1.0)).astype(np.float32)
    act = T(act_np)
    awq = deq(lib.cg_quantize_awq(w._ptr, act._ptr, 64))
    aerr = lambda wq: np.linalg.norm(act_np @ (wq - w_np).T)
    assert aerr(awq) <= aerr(plain) * 1.0001


def test_int4_kv_cache_counts_tokens_once_and_attention_matches_reference():
    lib = L()
    layers, heads, D, Hq = 2, 2, 8, 4
    cache = lib.cg_kv_cache_int4_new(layers, 16, heads, D, 4)
    for t in range(5):
        for layer in range(layers):
            k, v = T(rng.standard_normal((heads * D,), dtype=np.float32)), T(rng.standard_normal((heads * D,), dtype=np.float32))
            lib.cg_kv_cache_int4_append(cache, layer, k._ptr, v._ptr)
    assert cache.contents.current_len == 5                  # once per token, not once per (token, layer)
    k_out, v_out = cg.Tensor((5, heads, D)), cg.Tensor((5, heads, D))
    lib.cg_kv_cache_int4_get(cache, 1, k_out._ptr, v_out._ptr)
    q_np = rng.standard_normal((2, Hq * D), dtype=np.float32)
    q, out = T(q_np), cg.Tensor((2, Hq * D))
    lib.cg_attention_int4_kv(q._ptr, cache, 1, out._ptr)
    K = torch.tensor(k_out.numpy()).repeat_interleave(Hq // heads, 1)      # [5, Hq, D]
    V = torch.tensor(v_out.numpy()).repeat_interleave(Hq // heads, 1)
    Q = torch.tensor(q_np).view(2, Hq, D)
    s = torch.einsum("qhd,khd->hqk", Q, K) / D ** 0.5
    mask = torch.arange(5)[None, :] > (torch.arange(2)[:, None] + 3)
    s = s.masked_fill(mask[None], float("-inf"))
    ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), V).reshape(2, Hq * D)
    assert np.allclose(out.numpy(), ref.numpy(), atol=1e-5)
    lib.cg_kv_cache_int4_truncate(cache, 3)
    assert cache.contents.current_len == 3
    lib.cg_kv_cache_int4_free(cache)
    cal = lib.cg_calibration_new(4)
    a = T([[1, -2, 0.5, 0], [3, 1, -0.5, 0]])
    lib.cg_calibration_update(cal, a._ptr)
    scales, zeros = (c_float * 4)(), (c_float * 4)()
    lib.cg_calibration_compute_scales(cal, scales, zeros, 1)
    assert np.allclose(list(scales), [3 / 15, 3 / 15, 1 / 15, 1.0]) and list(zeros)[:2] == [0.0, 10.0]
    lib.cg_calibration_free(cal)


# --------------------------------------------------------------------- attention
@pytest.mark.parametrize("mask_type,hk", [(0, 4), (1, 4), (1, 2), (2, 1)])
def test_flash_attention_cpu_matches_torch(mask_type, hk):
    lib = L()
    B, Tq, Tk, H, D = 2, 5, 7, 4, 8
    q_np, k_np, v_np = (rng.standard_normal(s, dtype=np.float32) for s in ((B, Tq, H, D), (B, Tk, hk, D), (B, Tk, hk, D)))
    do_np = rng.standard_normal((B, Tq, H, D), dtype=np.float32)
    q, k, v, do = T(q_np), T(k_np), T(v_np), T(do_np)
    p = lib.cg_flash_attn_params_new(q._ptr, k._ptr, v._ptr, mask_type, 0.0)
    p.contents.window_size = 3
    p.contents.config.block_n = 4
    lib.cg_flash_attention_forward_cpu(p)
    p.contents.dO = do._ptr
    lib.cg_flash_attention_backward_cpu(p)
    tq, tk, tv = (torch.tensor(x, requires_grad=True) for x in (q_np, k_np, v_np))
    kk, vv = tk.repeat_interleave(H // hk, 2), tv.repeat_interleave(H // hk, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", tq, kk) / D ** 0.5
    rel = torch.arange(Tk)[None, :] - (torch.arange(Tq)[:, None] + Tk - Tq)
    if mask_type >= 1:
        s = s.masked_fill(rel > 0, float("-inf"))
    if mask_type == 2:
        s = s.masked_fill(-rel >= 3, float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)
    (o * torch.tensor(do_np)).sum().backward()
    assert np.allclose(borrowed(p.contents.O), o.detach().numpy(), atol=1e-5)
    assert np.allclose(borrowed(p.contents.L), torch.logsumexp(s, -1).detach().numpy(), atol=1e-5)
    for mine, ref in ((p.contents.dQ, tq), (p.contents.dK, tk), (p.contents.dV, tv)):
        assert np.allclose(borrowed(mine), ref.grad.numpy(), atol=1e-4)
    lib.cg_flash_attn_params_free(p)
    cfg = lib.cg_flash_attn_autotune(1, 8192, 128, 148)
    assert cfg.split_k == 64 and cfg.num_stages == 3 and lib.cg_flash_attn_autotune(2048, 2048, 64, 148).split_k == 1


def test_rope_and_alibi():
    lib = L()
    T_, H, D = 4, 2, 8
    q_np = rng.standard_normal((T_, H, D), dtype=np.float32)
    q = q_np.copy()
    lib.cg_apply_rope(q.ctypes.data_as(FP), None, T_, H, D, 3, 10000.0)
    pos = np.arange(3, 3 + T_, dtype=np.float32)[:, None] * (10000.0 ** (-2 * np.arange(D // 2, dtype=np.float32) / D))[None]
    c, s = np.cos(pos)[:, None, :], np.sin(pos)[:, None, :]
    ref = np.concatenate([q_np[..., :4] * c - q_np[..., 4:] * s, q_np[..., :4] * s + q_np[..., 4:] * c], -1)
    assert np.allclose(q, ref, atol=1e-5)
    slopes = (c_float * 8)()
    lib.cg_alibi_slopes(slopes, 8)
    assert np.allclose(list(slopes), [2.0 ** -(i + 1) for i in range(8)])


# ------------------------------------------------------------ sampling / decoding
def test_samplers_respect_their_support_and_distribution():
    lib = L()
    lib.cg_sample_seed(123)
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32))
    lp = logits.ctypes.data_as(FP)
    assert lib.cg_sample_temperature(lp, 4, 0.0) == 0
    draws = np.array([lib.cg_sample_temperature(lp, 4, 1.0) for _ in range(4000)])
    assert np.allclose(np.bincount(draws, minlength=4) / 4000, [0.5, 0.3, 0.15, 0.05], atol=0.03)
    assert {lib.cg_sample_top_k(lp, 4, 2) for _ in range(300)} == {0, 1}
    assert {lib.cg_sample_top_p(lp, 4, 0.75) for _ in range(300)} == {0, 1}
    assert {lib.cg_sample_top_p(lp, 4, 0.4) for _ in range(100)} == {0}
    assert set(lib.cg_sample_typical(lp, 4, 0.5) for _ in range(300)) <= {0, 1, 2}
    assert lib.cg_acceptance_prob(0.5, 0.25) == 0.5 and lib.cg_acceptance_prob(0.2, 0.9) == 1.0 and lib.cg_acceptance_prob(0.0, 0.1) == 1.0
    draft, target = np.array([0.7, 0.2, 0.1, 0.0], np.float32), np.array([0.4, 0.3, 0.1, 0.2], np.float32)
    draws = np.array([lib.cg_sample_corrected(draft.ctypes.data_as(FP), target.ctypes.data_as(FP), 4) for _ in range(3000)])
    assert np.allclose(np.bincount(draws, minlength=4) / 3000, [0, 1 / 3, 0, 2 / 3], atol=0.03)


def _toy_model(V, seed, sharpness):
    table = np.random.default_rng(seed).standard_normal((V, V)).astype(np.float32) * sharpness

    @LogitsFn
    def fn(_model, ids, length, n_pos, out):
        for j in range(n_pos):
            tok = ids[length - n_pos + j]
            for v in range(V):
                out[j * V + v] = table[tok % V, v]
    return fn, table


def test_speculative_decoding_equals_target_greedy_and_preserves_target_distribution():
    lib = L()
    V = 6
    target_fn, table = _toy_model(V, 5, 2.0)
    draft_fn, _ = _toy_model(V, 6, 2.0)
    dec = lib.cg_speculative_decoder_new(None, None, 3)
    lib.cg_speculative_set_models(dec, draft_fn, target_fn, V)
    prompt = T([1.0, 4.0])
    out = cg.Tensor.from_ptr(lib.cg_speculative_generate(dec, prompt._ptr, 12, 0.0, 1.0))
    ids = out.numpy().astype(int).tolist()
    want = [1, 4]
    for _ in range(12):
        want.append(int(table[want[-1]].argmax()))
    assert ids == want                                       # greedy: exactly the target's own decode
    assert dec.contents.num_steps >= 1 and 0.0 <= dec.contents.avg_acceptance_rate <= 1.0
    # identical models: every draft token is accepted
    same = lib.cg_speculative_decoder_new(None, None, 4)
    lib.cg_speculative_set_models(same, target_fn, target_fn, V)
    r = cg.Tensor.from_ptr(lib.cg_speculative_generate(same, prompt._ptr, 20, 1.0, 1.0))
    assert r.shape == (22,) and same.contents.avg_acceptance_rate == 1.0
    # sampling: the first generated token follows the target distribution although drafts come from another model
    counts = np.zeros(V)
    for trial in range(1500):
        dec.contents.rng_state = 1000 + trial
        r = cg.Tensor.from_ptr(lib.cg_speculative_generate(dec, prompt._ptr, 1, 1.0, 1.0))
        counts[int(r.numpy()[2])] += 1
    p = torch.softmax(torch.tensor(table[4]), -1).numpy()
    assert np.allclose(counts / 1500, p, atol=0.04)
    lib.cg_speculative_decoder_free(dec)
    lib.cg_speculative_decoder_free(same)


def test_token_tree_mask_and_eagle_tree():
    lib = L()
    tree = lib.cg_token_tree_new(3)
    lib.cg_token_tree_add_token(tree, 11, None)              # 0: child of the prefix
    lib.cg_token_tree_add_token(tree, 12, None)              # 1: child of 0
    assert lib.cg_token_tree_add_child(tree, 0, 13, None) == 2   # sibling branch under 0
    mask = cg.Tensor.from_ptr(lib.cg_tree_attention_mask(tree, 2))
    m = mask.numpy()[0, 0] == 0
    want = np.array([[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [1, 1, 1, 0, 0], [1, 1, 1, 1, 0], [1, 1, 1, 0, 1]], bool)
    assert mask.shape == (1, 1, 5, 5) and np.array_equal(m, want) and mask.numpy().min() == -1e9
    lib.cg_token_tree_free(tree)
    V = 8
    fn, table = _toy_model(V, 9, 1.0)
    dec = lib.cg_speculative_decoder_new(None, None, 3)
    lib.cg_speculative_set_models(dec, fn, fn, V)
    eagle = lib.cg_eagle_draft_new(dec)
    prompt = T([2.0])
    t = lib.cg_eagle_generate_tree(eagle, prompt._ptr, 3)
    c = t.contents
    assert c.depth == 3 and c.num_tokens >= 3
    parents = [c.parents[i] for i in range(c.num_tokens)]
    assert parents[0] == -1 and all(p < i for i, p in enumerate(parents))
    assert c.tokens[0] == int(table[2].argmax())             # the most probable token leads each level
    lib.cg_token_tree_free(t)
    lib.cg_eagle_draft_free(eagle)
    lib.cg_speculative_decoder_free(dec)


# ---------------------------------------------------------------------- pipeline
FWD, BWD, SEND_F, RECV_F, SEND_B, RECV_B, WAIT, SYNC, OPT = range(9)          # cg_schedule_op


@pytest.mark.parametrize("S,M", [(1, 1), (2, 4), (4, 8), (4, 2), (8, 8)])
def test_1f1b_schedule_properties(S, M):
    lib = L()
    for stage in range(S):
        n = c_int()
        steps = lib.cg_pipeline_gen_1f1b_stage(S, M, stage, byref(n))
        acts = [(steps[i].action, steps[i].microbatch_id) for i in range(n.value)]
        f = [m for a, m in acts if a == FWD]
        b = [m for a, m in acts if a == BWD]
        assert f == list(range(M)) and b == list(range(M)) and acts[-1][0] == OPT
        in_flight = peak = 0
        done_f = set()
        for a, m in acts:
            if a == FWD:
                in_flight += 1
                done_f.add(m)
            if a == BWD:
                assert m in done_f
                in_flight -= 1
            peak = max(peak, in_flight)
        assert peak == min(S - stage, M)                     # bounded activation memory
        assert sum(a == RECV_F for a, _ in acts) == (M if stage > 0 else 0)
        assert sum(a == SEND_B for a, _ in acts) == (M if stage > 0 else 0)
        assert sum(a == SEND_F for a, _ in acts) == (M if stage < S - 1 else 0)
        ctypes.CDLL(None).free(ctypes.cast(steps, c_void_p))
    n = c_int()
    steps = lib.cg_pipeline_gen_interleaved_stage(2, 2, 4, 0, byref(n))
    acts = [(steps[i].action, steps[i].microbatch_id, steps[i].stage_id) for i in range(n.value)]
    assert sum(a == FWD for a, _, _ in acts) == 8 and sum(a == BWD for a, _, _ in acts) == 8
    assert {s for a, _, s in acts if a == FWD} == {0, 2}     # virtual stages chunk * S + rank


def test_pipeline_executor_matches_single_stage_gradients():
    lib = L()
    lib.cg_manual_seed(11)
    layers = [lib.cg_linear_new(6, 8, True), lib.cg_tanh_new(), lib.cg_linear_new(8, 8, True), lib.cg_relu_new(), lib.cg_linear_new(8, 3, True)]
    stages = [lib.cg_sequential_new() for _ in range(3)]
    for l, s in zip(layers, [0, 0, 1, 1, 2]):
        lib.cg_sequential_add(stages[s], l)
    x_np, y_np = rng.standard_normal((8, 6), dtype=np.float32), rng.standard_normal((8, 3), dtype=np.float32)
    x, y = T(x_np), T(y_np)
    pp = lib.cg_pipeline_new(3, 4)
    for i, s in enumerate(stages):
        lib.cg_pipeline_set_stage(pp, i, s, 1)
    lib.cg_pipeline_forward_backward(pp, x._ptr, y._ptr)
    assert lib.cg_last_error() == 0
    ws = [torch.tensor(borrowed(layers[i].contents.weights), requires_grad=True) for i in (0, 2, 4)]
    bs = [torch.tensor(borrowed(layers[i].contents.bias), requires_grad=True) for i in (0, 2, 4)]
    h = torch.tanh(torch.tensor(x_np) @ ws[0] + bs[0])
    h = torch.relu(h @ ws[1] + bs[1])
    out = h @ ws[2] + bs[2]
    loss = sum(torch.nn.functional.mse_loss(out[i * 2:(i + 1) * 2], torch.tensor(y_np[i * 2:(i + 1) * 2])) for i in range(4)) / 4
    loss.backward()
    assert abs(pp.contents.last_loss - loss.item()) < 1e-5
    for i, (w, b) in zip((0, 2, 4), zip(ws, bs)):
        assert np.allclose(grad_of(layers[i].contents.weights), w.grad.numpy(), atol=1e-5)
        assert np.allclose(grad_of(layers[i].contents.bias), b.grad.numpy(), atol=1e-5)
    lib.cg_pipeline_free(pp)
    for s in stages:
        lib.cg_sequential_free(s)


def test_3d_rank_mapping():
    lib = L()
    ctx = lib.cg_3d_parallel_new(2, 2, 2)
    lib.cg_3d_parallel_init_from_world(ctx, 8, 5)
    c = ctx.contents
    assert (c.tp_rank, c.pp_rank, c.dp_rank) == (1, 0, 1)
    assert [c.tp_group.contents.ranks[i] for i in range(2)] == [4, 5]
    assert [c.pp_group.contents.ranks[i] for i in range(2)] == [5, 7]
    assert [c.dp_group.contents.ranks[i] for i in range(2)] == [1, 5]
    lib.cg_3d_parallel_free(ctx)


# ------------------------------------------------------------------------ memory
def test_pool_buddy_planner():
    lib = L()
    assert [lib.cg_subbin_index(s) for s in (768, 1024, 4096, 1000)] == [0, 1, 2, -1]
    pool = lib.cg_memory_pool_new()
    a = lib.cg_pool_alloc(pool, 768)
    lib.cg_pool_free(pool, a)
    assert lib.cg_pool_alloc(pool, 768) == a                 # exact-size sub-bin reuse
    b = lib.cg_pool_alloc(pool, 3 << 30 >> 20)               # 3 KiB -> 4 KiB bin
    c = lib.cg_pool_alloc(pool, 5000)
    lib.cg_pool_free(pool, b)
    lib.cg_pool_free(pool, c)
    assert 0.0 < lib.cg_memory_fragmentation(pool) < 1.0
    lib.cg_pool_trim(pool)
    lib.cg_memory_pool_free(pool)
    slab = ctypes.create_string_buffer(1 << 16)
    base = ctypes.addressof(slab)
    buddy = lib.cg_buddy_new(base, 1 << 16)
    p1, p2 = lib.cg_buddy_alloc(buddy, 1000), lib.cg_buddy_alloc(buddy, 1000)
    assert p1 == base and p2 == base + 1024 and lib.cg_buddy_splits(buddy) == 6
    lib.cg_buddy_free(buddy, p1, 1000)
    lib.cg_buddy_free(buddy, p2, 1000)
    assert lib.cg_buddy_coalesces(buddy) == 6 and lib.cg_buddy_alloc(buddy, 1 << 16) == base
    assert not lib.cg_buddy_alloc(buddy, 256)
    lib.cg_buddy_destroy(buddy)


def _chain_graph(lib, n_ops=6, size=1024):
    """x -> exp -> relu -> ... chain of unary ops built by tracing the eager API."""
    ts = [cg.Tensor((size,)) for _ in range(n_ops + 1)]
    ts[0].numpy()[:] = rng.standard_normal(size)
    lib.cg_jit_begin_trace()
    for i in range(n_ops):
        lib.cg_tensor_exp(ts[i]._ptr, ts[i + 1]._ptr) if i % 2 == 0 else lib.cg_tensor_add(ts[i]._ptr, ts[i]._ptr, ts[i + 1]._ptr)
    return lib.cg_jit_end_trace(), ts


def test_memory_planner_reuses_dead_tensors_and_replays_addresses():
    lib = L()
    g, ts = _chain_graph(lib)
    planner = lib.cg_memory_planner_new()
    lib.cg_memory_plan_analyze(planner, g)
    assert lib.cg_memory_plan_bytes(planner) <= 4 * 4096     # 5 intermediates of 4 KiB share storage (+ pinned ends)
    assert lib.cg_can_reuse_memory(planner, 1, 3) and not lib.cg_can_reuse_memory(planner, 1, 2)
    lib.cg_cuda_graph_capture_begin(planner)
    first = [lib.cg_planned_alloc(planner, 4096, i) for i in (1, 2, 3)]
    lib.cg_cuda_graph_capture_end(planner)
    assert first[0] == first[2] and first[0] != first[1] and not lib.cg_cuda_graph_needs_update(planner)
    lib.cg_cuda_graph_replay(planner)
    assert [lib.cg_planned_alloc(planner, 4096, i) for i in (1, 2, 3)] == first
    lib.cg_cuda_graph_replay(planner)
    lib.cg_planned_alloc(planner, 4096, 4)                   # deviates from the captured sequence
    assert lib.cg_cuda_graph_needs_update(planner)
    lib.cg_memory_planner_free(planner)
    lib.cg_ir_graph_free(g)


# ---------------------------------------------------------------------- symbolic
def test_symbolic_shapes():
    lib = L()
    B, S = lib.cg_dim_var(b"batch"), lib.cg_dim_var(b"seq")
    lib.cg_dim_constrain(S, 1, 4096)
    a = lib.cg_shape_new((c_void_p * 3)(B, S, lib.cg_dim_const(64)), 3)
    w = lib.cg_shape_from_ints((c_int * 2)(64, 256), 2)
    out = lib.cg_shape_matmul(a, w)
    assert lib.cg_shape_is_dynamic(out)
    names, vals, dims = (c_char_p * 2)(b"batch", b"seq"), (c_int64 * 2)(8, 128), (c_int * 3)()
    assert lib.cg_shape_resolve(out, vals, names, 2, dims) and list(dims) == [8, 128, 256]
    vals[1] = 5000
    assert not lib.cg_shape_resolve(out, vals, names, 2, dims)      # violates the constraint on seq
    assert not lib.cg_shape_matmul(a, lib.cg_shape_from_ints((c_int * 2)(32, 256), 2)) and lib.cg_last_error() == 2
    e = lib.cg_expr_floordiv(lib.cg_expr_mul(lib.cg_expr_var(b"seq"), lib.cg_expr_const(3)), lib.cg_expr_add(lib.cg_expr_const(1), lib.cg_expr_const(1)))
    assert take_string(lib.cg_expr_to_string(e)) == "((seq * 3) // 2)"
    d = lib.cg_dim_inferred(e)
    half = lib.cg_shape_new((c_void_p * 1)(d), 1)
    vals[1] = 10
    one = (c_int * 1)()
    assert lib.cg_shape_resolve(half, vals, names, 2, one) and one[0] == 15
    spec = lib.cg_shape_specialize(out, vals, names, 2)
    assert lib.cg_shape_guards_hold(spec, vals, names, 2)
    vals[0] = 9
    assert not lib.cg_shape_guards_hold(spec, vals, names, 2)
    assert lib.cg_shape_hash(out) != lib.cg_shape_hash(a)
    lib.cg_shape_specialization_free(spec)
    for s in (a, w, out, half):
        lib.cg_shape_free(s)


# --------------------------------------------------------------------------- JIT
def test_trace_cse_dce_codegen_and_compiled_module_match_eager():
    lib = L()
    n = 257
    a, b = T(rng.standard_normal(n, dtype=np.float32)), T(rng.standard_normal(n, dtype=np.float32))
    s1, s2, prod, dead, out = (cg.Tensor((n,)) for _ in range(5))
    lib.cg_jit_begin_trace()
    lib.cg_tensor_add(a._ptr, b._ptr, s1._ptr)
    lib.cg_tensor_add(b._ptr, a._ptr, s2._ptr)               # same value as s1 (commutative)
    lib.cg_tensor_mul(s1._ptr, s2._ptr, prod._ptr)
    lib.cg_tensor_exp(a._ptr, dead._ptr)                     # result unused
    lib.cg_tensor_exp(prod._ptr, out._ptr)
    g = lib.cg_jit_end_trace()
    want = np.exp((a.numpy() + b.numpy()) ** 2)
    assert g.contents.num_nodes == 5
    lib.cg_ir_graph_mark_output(g, out._ptr)
    # `dead` was auto-marked as an output because nothing consumed it: drop it to test DCE
    g.contents.num_outputs = 0
    lib.cg_ir_graph_mark_output(g, out._ptr)
    lib.cg_ir_optimize(g, 2)
    assert lib.cg_ir_graph_live_nodes(g) == 3                # one add removed by CSE, the stray exp by DCE
    out.numpy()[:] = 0
    assert lib.cg_ir_execute(g) and np.allclose(out.numpy(), want, rtol=1e-5)
    src = take_string(lib.cg_jit_codegen_c(g))
    assert src.count("for (long i") == 1 and "expf" in src   # the three ops share one loop
    cu = take_string(lib.cg_jit_codegen_cuda(g))
    assert 'extern "C" __global__ void jit_kernel(float* const* t, long n)' in cu and cu.count("t[") == 3   # 2 loads, 1 store
    comp = lib.cg_jit_compiler_new(g, 0)
    compiled = lib.cg_jit_compile(comp)
    out.numpy()[:] = 0
    assert lib.cg_jit_run(comp) and np.allclose(out.numpy(), want, rtol=1e-5)
    import shutil
    assert compiled == (shutil.which("cc") is not None)
    lib.cg_jit_compiler_free(comp)
    bad = lib.cg_jit_compiler_new(g, 2)
    assert not lib.cg_jit_compile(bad)                       # Metal: unsupported backend
    lib.cg_jit_compiler_free(bad)
    lib.cg_ir_graph_free(g)


def test_fusion_patterns_and_attention_rewrite():
    lib = L()
    OP = {"add": 1, "relu": 10, "gelu": 13, "softmax": 14, "matmul": 15, "ln": 27}
    g = lib.cg_ir_graph_new()
    q, kt, v = T(rng.standard_normal((4, 8), dtype=np.float32)), T(rng.standard_normal((8, 6), dtype=np.float32)), T(rng.standard_normal((6, 8), dtype=np.float32))
    w, bias = T(rng.standard_normal((8, 8), dtype=np.float32)), T(rng.standard_normal((4, 8), dtype=np.float32))
    s, p, o, h, hb, y = (cg.Tensor(sh) for sh in ((4, 6), (4, 6), (4, 8), (4, 8), (4, 8), (4, 8)))
    tid = lambda t: lib.cg_ir_graph_tensor_id(g, t._ptr)
    node = lambda op, ins, out: lib.cg_ir_graph_add_node(g, OP[op], (c_int * len(ins))(*[tid(t) for t in ins]), len(ins), tid(out), None, 0)
    node("matmul", [q, kt], s); node("softmax", [s], p); node("matmul", [p, v], o)
    node("matmul", [o, w], h); node("add", [h, bias], hb); node("relu", [hb], y)
    lib.cg_ir_graph_mark_output(g, y._ptr)
    assert lib.cg_ir_execute(g)
    want = y.numpy().copy()
    ref = torch.relu(torch.softmax(torch.tensor(q.numpy() @ kt.numpy()), -1) @ torch.tensor(v.numpy()) @ torch.tensor(w.numpy()) + torch.tensor(bias.numpy()))
    assert np.allclose(want, ref.numpy(), atol=1e-5)
    fp = lib.cg_fusion_pass_new(g)
    lib.cg_fusion_analyze(fp)
    groups = [fp.contents.groups[i].contents for i in range(fp.contents.num_groups)]
    assert [(gr.kernel_name, gr.fusion_type, gr.num_nodes) for gr in groups] == [(b"fused_attention", 4, 3), (b"fused_matmul_epilogue", 3, 3)]
    assert groups[1].memory_saved == 2 * 2 * 4 * 32
    plan = take_string(lib.cg_fusion_generate_kernel(fp.contents.groups[1]))
    assert "bias -> relu" in plan
    lib.cg_fusion_apply(fp)
    assert lib.cg_ir_graph_live_nodes(g) == 4                # attention collapsed into one node
    y.numpy()[:] = 0
    assert lib.cg_ir_execute(g) and np.allclose(y.numpy(), want, atol=1e-6)
    lib.cg_fusion_pass_free(fp)
    lib.cg_ir_graph_free(g)
