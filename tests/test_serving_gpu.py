"""Serving kernels on the GPU against their host restatements (fp32 PyTorch / the C library)."""
import pytest
import torch

from cogito_b200.models.llama import Llama, LlamaConfig
from cogito_b200.ops import _lib
from cogito_b200.quant.int4 import Int4Linear, dequantize_int4, quantize_int4
from cogito_b200.serve.engine import LlamaInt4Engine, SpeculativeDecoder
from cogito_b200.serve.kv_cache import PagedKVCacheInt4
from cogito_b200.serve.sampling import filtered_probs, sample, spec_accept, tree_attention_mask
from cogito_b200.utils import rng

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_int4_quantize_dequantize_bit_exact_with_host():
    torch.manual_seed(0)
    x = torch.randn(64, 384) * 2
    x[0, :4] = torch.tensor([0.5, 1.5, -0.5, -2.5]) * (x[0, :128].abs().max() / 7)
    pc, sc = quantize_int4(x, 128)
    pg, sg = quantize_int4(x.to(DEV), 128)
    assert torch.equal(pg.cpu(), pc) and torch.equal(sg.cpu(), sc)
    assert torch.equal(dequantize_int4(pg, sg, x.numel(), 128).cpu(), dequantize_int4(pc, sc, x.numel(), 128))
    assert torch.equal(dequantize_int4(pg, sg, x.numel(), 128, torch.bfloat16).cpu(),
                       dequantize_int4(pc, sc, x.numel(), 128).bfloat16())


@pytest.mark.parametrize("M,K,N,group,splits", [(16, 512, 256, 128, 0), (80, 1024, 384, 128, 2), (5, 256, 128, 64, 1),
                                                (130, 512, 256, 128, 0), (1, 4096, 512, 128, 0)])
@pytest.mark.parametrize("kernel", ["wb", "wa"])
def test_int4_gemm_matches_dequantised_product(M, K, N, group, splits, kernel):
    torch.manual_seed(M + K)
    w = torch.randn(N, K) * 0.05
    bias = torch.randn(N) * 0.1
    lin = Int4Linear(w, bias, group).to(DEV)
    lin.kernel = kernel
    x = (torch.randn(M, K) + 0.5).bfloat16()                # a DC offset exercises the row-sum correction of "wa"
    got = lin(x.to(DEV), splits=splits).float().cpu()
    # oracle: the same packed weights, dequantised on the host, fp32 product
    wt = dequantize_int4(lin.packed.cpu(), lin.scales.cpu(), K * N, group).view(K, N)
    ref = x.float() @ wt + lin.bias.float().cpu()
    err = (got - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
    _lib.assert_device_ok()


@pytest.mark.parametrize("D,group,Hk,Hq,Tq", [(128, 32, 2, 8, 5), (64, 16, 1, 4, 1), (128, 128, 2, 2, 3),
                                                 (128, 64, 2, 16, 5), (128, 32, 1, 4, 40), (128, 16, 1, 2, 2)])
def test_kv_append_and_attention_match_host(D, group, Hk, Hq, Tq):
    torch.manual_seed(D + Tq)
    B, hist = 3, 150
    gpu = PagedKVCacheInt4(2, B, 256, Hk, D, group, page_size=16, device=DEV)
    cpu = PagedKVCacheInt4(2, B, 256, Hk, D, group, page_size=16)
    perm = torch.randperm(gpu.page_table.numel()).view_as(gpu.page_table).int()
    gpu.page_table.copy_(perm); cpu.page_table.copy_(perm)
    k, v = torch.randn(B, hist, Hk, D).bfloat16(), torch.randn(B, hist, Hk, D).bfloat16()
    for c, d in ((gpu, DEV), (cpu, "cpu")):
        c.append(1, k.to(d), v.to(d))
        c.commit(torch.tensor([hist, hist - 7, hist - 33], dtype=torch.int32, device=d))
    assert torch.equal(gpu.k_pages[1].cpu(), cpu.k_pages[1]) and torch.equal(gpu.v_scales[1].cpu(), cpu.v_scales[1])
    kn, vn, q = (torch.randn(B, Tq, h, D).bfloat16() for h in (Hk, Hk, Hq))
    for c, d in ((gpu, DEV), (cpu, "cpu")):
        c.append(1, kn.to(d), vn.to(d))
    for splits in (1, 4):
        got = gpu.attention(1, q.to(DEV), splits=splits).float().cpu()
        ref = cpu.attention(1, q.float())
        assert (got - ref).abs().max().item() < 2e-2
    _lib.assert_device_ok()


def test_kv_attention_long_history_many_key_blocks():
    torch.manual_seed(3)
    B, hist, Hk, Hq, D, Tq = 2, 700, 2, 8, 128, 5
    gpu = PagedKVCacheInt4(1, B, 1024, Hk, D, 32, page_size=32, device=DEV)
    cpu = PagedKVCacheInt4(1, B, 1024, Hk, D, 32, page_size=32)
    k, v = torch.randn(B, hist, Hk, D).bfloat16(), torch.randn(B, hist, Hk, D).bfloat16()
    for c, d in ((gpu, DEV), (cpu, "cpu")):
        c.append(0, k.to(d), v.to(d))
        c.commit(torch.tensor([hist, hist - 301], dtype=torch.int32, device=d))
    kn, vn, q = (torch.randn(B, Tq, h, D).bfloat16() for h in (Hk, Hk, Hq))
    for c, d in ((gpu, DEV), (cpu, "cpu")):
        c.append(0, kn.to(d), vn.to(d))
    ref = cpu.attention(0, q.float())
    for splits in (1, 3, 0):
        got = gpu.attention(0, q.to(DEV), splits=splits).float().cpu()
        assert (got - ref).abs().max().item() < 2e-2
    _lib.assert_device_ok()


def test_sampling_matches_filtered_distribution():
    torch.manual_seed(1)
    V, rows = 32000, 4
    logits = torch.randn(rows, V) * 3
    for temp, k, p in ((1.0, 50, 0.9), (0.7, 8, 1.0), (1.3, 0, 0.5), (0.0, 50, 0.9)):
        tok, probs = sample(logits.to(DEV), temp, k, p, seed=5, step=0, return_probs=True)
        ref = filtered_probs(logits, temp, k, p)
        assert torch.allclose(probs.cpu(), ref, atol=2e-5), (temp, k, p)
        assert (ref.gather(1, tok.cpu().long()[:, None]) > 0).all()
    counts = torch.zeros(rows, V)
    step = torch.zeros(1, dtype=torch.int64, device=DEV)
    lg = logits.to(DEV).bfloat16()
    ref = filtered_probs(lg.float().cpu(), 1.0, 8, 1.0)
    for i in range(1500):
        step.fill_(i)
        counts.scatter_add_(1, sample(lg, 1.0, 8, 1.0, seed=9, step=step).cpu().long()[:, None], torch.ones(rows, 1))
    assert (counts / 1500 - ref).abs().max().item() < 0.05
    # different rows and steps draw from different streams
    same = torch.zeros(64, 1000, device=DEV)
    toks = sample(same, 1.0, 0, 1.0, seed=1, step=3)
    assert toks.unique().numel() > 32


def test_spec_accept_rule_and_commit():
    B, g, V = 64, 4, 512
    torch.manual_seed(2)
    q = torch.softmax(torch.randn(B, g, V), -1)
    p = torch.softmax(torch.randn(B, g + 1, V), -1)
    draft = torch.multinomial(q.view(-1, V), 1).view(B, g).int()
    # identical distributions: everything is accepted and a bonus token follows
    lengths = torch.full((B,), 10, dtype=torch.int32, device=DEV)
    stats = torch.zeros(2, dtype=torch.int32, device=DEV)
    pp = torch.cat([q, p[:, -1:]], 1)
    n, out = spec_accept(draft.to(DEV), q.to(DEV), pp.to(DEV), seed=1, step=0, lengths=lengths, stats=stats)
    assert (n == g).all() and torch.equal(out[:, :g].cpu(), draft) and (lengths == 10 + g + 1).all()
    assert stats.tolist() == [B * g, B * g]
    # zero target probability on the drafted token: rejected at position 0, resampled where p > q
    p0 = p.clone()
    p0[torch.arange(B), 0, draft[:, 0].long()] = 0
    p0[:, 0] /= p0[:, 0].sum(-1, keepdim=True)
    n, out = spec_accept(draft.to(DEV), q.to(DEV), p0.to(DEV), seed=1, step=1)
    assert (n == 0).all()
    tok = out[:, 0].cpu().long()
    assert ((p0[torch.arange(B), 0, tok] - q[torch.arange(B), 0, tok]) > 0).all()
    # acceptance frequency = E[min(1, p/q)] at the first position
    trials, acc0 = 300, 0
    for s in range(trials):
        n, _ = spec_accept(draft.to(DEV), q.to(DEV), p.to(DEV), seed=3, step=s)
        acc0 += (n >= 1).float().mean().item()
    ratio = (p[torch.arange(B), 0, draft[:, 0].long()] / q[torch.arange(B), 0, draft[:, 0].long()]).clamp(max=1).mean().item()
    assert abs(acc0 / trials - ratio) < 0.04
    parents = torch.tensor([-1, 0, 0, 2, 1], dtype=torch.int32)
    assert torch.equal(tree_attention_mask(parents.to(DEV), 7).cpu(), tree_attention_mask(parents, 7))


def test_engine_and_speculative_decoding_on_gpu():
    rng.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1024, n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, max_seq_len=256)
    target = Llama(cfg)
    B = 4
    cpu_engine = LlamaInt4Engine(target, B, 128)
    gpu_engine = LlamaInt4Engine(target.to(DEV).bfloat16(), B, 128)
    prompts = torch.randint(0, 1024, (B, 9))
    lc = cpu_engine.forward(prompts, commit=True)
    lg = gpu_engine.forward(prompts.to(DEV), commit=True).cpu()
    assert torch.nn.functional.cosine_similarity(lc.flatten(), lg.flatten(), dim=0) > 0.98
    draft_engine = LlamaInt4Engine(target, B, 128)          # same weights: all drafts accepted under greedy decoding
    sd = SpeculativeDecoder(draft_engine, gpu_engine, gamma=4, temperature=0.0)
    seqs, stats = sd.generate(prompts.to(DEV), 10)
    assert stats.acceptance_rate > 0.8 and all(len(s) >= 19 for s in seqs)   # < 1 only through bf16 near-ties
    _lib.assert_device_ok()
