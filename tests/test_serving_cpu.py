"""Serving stack on the host path: INT4 packing against the C library, paged KV cache,
sampling composition, speculative decoding."""
import numpy as np
import torch

from capi_defs import L, T, cg
from cogito_b200.models.llama import Llama, LlamaConfig, llama_tiny
from cogito_b200.quant.int4 import Int4Linear, dequantize_int4, quantize_int4
from cogito_b200.serve.engine import LlamaInt4Engine, SpeculativeDecoder
from cogito_b200.serve.kv_cache import PagedKVCacheInt4
from cogito_b200.serve.sampling import filtered_probs, sample, spec_accept, tree_attention_mask
from cogito_b200.utils import rng


def test_python_packing_is_bit_exact_with_the_c_library():
    lib = L()
    x = torch.randn(8, 96) * 3
    x[0, :4] = torch.tensor([0.5, 1.5, -0.5, -2.5]) * (x[0, :32].abs().max() / 7)     # exact halves: rounding away from zero
    packed, scales = quantize_int4(x, 32)
    xt = T(x.numpy())
    q = lib.cg_quantize_int4(xt._ptr, 32)
    assert np.array_equal(packed.numpy(), np.ctypeslib.as_array(q.contents.data, shape=(packed.numel(),)))
    assert np.array_equal(scales.numpy(), np.ctypeslib.as_array(q.contents.scales, shape=(scales.numel(),)))
    deq = cg.Tensor.from_ptr(lib.cg_dequantize(q))
    assert np.array_equal(dequantize_int4(packed, scales, x.numel(), 32).view(8, 96).numpy(), deq.numpy())
    lib.cg_tensor_quant_free(q)
    lin = Int4Linear(torch.randn(128, 64), torch.randn(128), group=64)
    xin = torch.randn(3, 64)
    assert torch.allclose(lin(xin), xin @ lin.dequantized() + lin.bias.float(), atol=1e-5)


def test_paged_cache_matches_contiguous_attention_and_rolls_back():
    torch.manual_seed(0)
    B, H, Hq, D = 2, 2, 4, 16
    cache = PagedKVCacheInt4(2, B, 40, H, D, group=8, page_size=8)
    cache.page_table = cache.page_table.flip(1).contiguous()          # any placement works
    ks, vs = [], []
    for step, T_ in enumerate((9, 1, 3)):
        k, v = torch.randn(B, T_, H, D), torch.randn(B, T_, H, D)
        for layer in range(2):
            cache.append(layer, k, v)
        cache.commit(T_)
        ks.append(k); vs.append(v)
    assert cache.lengths.tolist() == [13, 13]
    k_all = torch.cat(ks, 1)
    kd, vd = cache.gather(1, 0, 13)
    assert (kd - k_all[0].bfloat16().float()).abs().max() <= k_all[0].abs().max() / 14 + 1e-3
    # verify pass: 3 new tokens, accept only 1 -> the other two positions are overwritten next time
    k, v, q = torch.randn(B, 3, H, D), torch.randn(B, 3, H, D), torch.randn(B, 3, Hq, D)
    cache.append(0, k, v)
    out = cache.attention(0, q)
    kd, vd = cache.gather(0, 1, 16)
    kk, vv = kd.repeat_interleave(2, 1), vd.repeat_interleave(2, 1)
    s = torch.einsum("qhd,khd->hqk", q[1].bfloat16().float(), kk) / D ** 0.5      # queries are bf16 on every path
    s = s.masked_fill((torch.arange(16)[None] > torch.arange(3)[:, None] + 13)[None], float("-inf"))
    assert torch.allclose(out[1], torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv), atol=1e-5)
    cache.commit(torch.tensor([1, 2], dtype=torch.int32))
    assert cache.lengths.tolist() == [14, 15]


def test_sampling_composition_and_acceptance_rule():
    logits = torch.log(torch.tensor([[0.4, 0.3, 0.2, 0.06, 0.04]]))
    p = filtered_probs(logits, 1.0, top_k=4, top_p=0.8)
    assert torch.allclose(p, torch.tensor([[0.4, 0.3, 0.2, 0.0, 0.0]]) / 0.9, atol=1e-6)
    assert torch.equal(filtered_probs(logits, 0.0), torch.tensor([[1.0, 0, 0, 0, 0]]))
    cold = filtered_probs(logits, 0.5, 0, 1.0)
    assert cold[0, 0] > 0.4 and abs(float(cold.sum()) - 1) < 1e-6
    toks = torch.stack([sample(logits, 1.0, 4, 0.8, seed=3, step=i) for i in range(3000)]).view(-1)
    freq = torch.bincount(toks.long(), minlength=5) / 3000.0
    assert torch.allclose(freq, p[0], atol=0.03)
    # acceptance: q puts all mass on token 0, p half on 0 and half on 2 -> accept w.p. 0.5, else resample 2
    q = torch.tensor([[[1.0, 0, 0]]]); pt = torch.tensor([[[0.5, 0, 0.5], [0, 1.0, 0]]])
    draft = torch.zeros(1, 1, dtype=torch.int32)
    gen = torch.Generator().manual_seed(0)
    acc = 0
    for _ in range(2000):
        n, out = spec_accept(draft, q, pt, generator=gen)
        acc += int(n[0])
        assert out[0].tolist() == ([0, 1] if int(n[0]) == 1 else [2, 0])
    assert abs(acc / 2000 - 0.5) < 0.04
    mask = tree_attention_mask(torch.tensor([-1, 0, 0], dtype=torch.int32), 2)
    want = torch.tensor([[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [1, 1, 1, 0, 0], [1, 1, 1, 1, 0], [1, 1, 1, 0, 1]], dtype=torch.bool)
    assert torch.equal(mask == 0, want)


def _greedy(engine, prompts, n):
    B = prompts.shape[0]
    engine.reset()
    cur = engine.forward(prompts, commit=True)[:, -1].argmax(-1)
    seqs = [prompts[b].tolist() for b in range(B)]
    for _ in range(n):
        for b in range(B):
            seqs[b].append(int(cur[b]))
        cur = engine.forward(cur.view(B, 1), commit=True)[:, 0].argmax(-1)
    return seqs


def test_speculative_decoding_reproduces_target_greedy_and_accepts_its_own_drafts():
    rng.manual_seed(0)
    target = Llama(llama_tiny())
    draft = Llama(LlamaConfig(vocab_size=256, n_layer=1, d_model=128, n_head=2, n_kv_head=1, d_ff=256, max_seq_len=256))
    B = 2
    te, de = LlamaInt4Engine(target, B, 128), LlamaInt4Engine(draft, B, 128)
    prompts = torch.randint(0, 256, (B, 5))
    want = _greedy(te, prompts, 12)
    got, stats = SpeculativeDecoder(de, te, gamma=3, temperature=0.0).generate(prompts, 12)
    for b in range(B):
        assert got[b][:17] == want[b][:17]
    # the target as its own draft: every token accepted, gamma + 1 tokens per step, still the same text
    te2 = LlamaInt4Engine(target, B, 128)
    got2, stats2 = SpeculativeDecoder(te2, te, gamma=3, temperature=0.0).generate(prompts, 12)
    assert stats2.acceptance_rate == 1.0 and stats2.steps == 3
    for b in range(B):
        assert got2[b][:17] == want[b][:17]
    # the engine agrees with the training model up to quantisation error
    te.reset()
    logits = te.forward(prompts, commit=True)
    ref = target(prompts).float()
    assert torch.nn.functional.cosine_similarity(logits.flatten(), ref.flatten(), dim=0) > 0.9


def test_engine_round_trips_through_a_quantised_checkpoint(tmp_path):
    from cogito_b200.io.checkpoint import load_tensors
    rng.manual_seed(2)
    cfg = LlamaConfig(vocab_size=256, n_layer=2, d_model=128, n_head=4, n_kv_head=2, d_ff=256, max_seq_len=64)
    eng = LlamaInt4Engine(Llama(cfg), batch=2, weight_group=64, kv_group=16, page_size=8)
    path = str(tmp_path / "engine.cog")
    nbytes = eng.save(path)
    st = load_tensors(path)
    assert st["layers.0.qkv"].dtype == torch.uint8 and st["layers.0.qkv.scales"].dtype == torch.float32
    assert nbytes < sum(p.numel() for p in Llama(cfg).parameters()) * 4 * 0.5      # nibbles + scales + bf16/fp32 embedding
    back = LlamaInt4Engine.load(path, cfg, batch=2, weight_group=64, kv_group=16, page_size=8)
    ids = torch.randint(0, 256, (2, 7))
    assert torch.equal(eng.forward(ids, commit=True), back.forward(ids, commit=True))
    nxt = torch.randint(0, 256, (2, 1))
    assert torch.equal(eng.forward(nxt), back.forward(nxt))
