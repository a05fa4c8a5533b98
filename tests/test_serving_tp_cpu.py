"""Tensor-parallel INT4 serving on CPU ranks (gloo): a TP=2 engine must produce the logits of the
unsplit engine, and speculative decoding must emit the same tokens on every rank."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cogito_b200.models.llama import Llama, LlamaConfig
        from cogito_b200.serve.engine import LlamaInt4Engine, SpeculativeDecoder
        from cogito_b200.utils.rng import manual_seed
        manual_seed(0)
        # vocabulary 384: slices of 256 per rank, the second one half padding
        cfg = LlamaConfig(vocab_size=384, n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, max_seq_len=64)
        # the draft's 192 hidden units are three weight groups: the ranks hold two and one of them
        dcfg = LlamaConfig(vocab_size=384, n_layer=1, d_model=256, n_head=4, n_kv_head=2, d_ff=192, max_seq_len=64)
        target, draft = Llama(cfg), Llama(dcfg)
        group = dist.new_group(list(range(world)))
        # weight groups of 64 = one head: every slice is cut on group boundaries, so the split engines hold
        # exactly the quantised values of the unsplit one
        one = LlamaInt4Engine(target, batch=2, weight_group=64, kv_group=32, page_size=16)
        tp = LlamaInt4Engine(target, batch=2, weight_group=64, kv_group=32, page_size=16, tp_group=group)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, 384, (2, 9), generator=g)
        a, b = one.forward(prompt, commit=True), tp.forward(prompt, commit=True)
        err1 = (a - b).abs().max().item()
        nxt = torch.randint(0, 384, (2, 3), generator=g)
        err2 = (one.forward(nxt) - tp.forward(nxt)).abs().max().item()
        sizes = (tp.lm_head.out_features, tp.cache.heads, tp.layers[0]["qkv"].out_features, tp.layers[0]["down"].in_features)
        dec = SpeculativeDecoder(LlamaInt4Engine(draft, batch=2, weight_group=64, kv_group=32, page_size=16, tp_group=group),
                                 LlamaInt4Engine(target, batch=2, weight_group=64, kv_group=32, page_size=16, tp_group=group),
                                 gamma=3, temperature=0.8, top_k=20, top_p=0.9, seed=5)
        ref = SpeculativeDecoder(LlamaInt4Engine(draft, batch=2, weight_group=64, kv_group=32, page_size=16),
                                 LlamaInt4Engine(target, batch=2, weight_group=64, kv_group=32, page_size=16),
                                 gamma=3, temperature=0.8, top_k=20, top_p=0.9, seed=5)
        out, _ = dec.generate(prompt, 12)
        out_ref, _ = ref.generate(prompt, 12)
        q.put((rank, err1, err2, sizes, out, out_ref, float(a.abs().max())))
    finally:
        dist.destroy_process_group()


def test_tp2_engine_matches_the_unsplit_engine():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err1, err2, sizes, out, out_ref, scale in res:
        assert sizes == (256, 1, (2 + 1 + 1) * 64, 256)
        assert err1 < 1e-3 * max(1.0, scale) and err2 < 1e-3 * max(1.0, scale), (err1, err2)
    assert res[0][4] == res[1][4]                      # both ranks emit the same tokens
    # the split engines follow the unsplit decoder (same random stream; the sums differ only in order)
    same = sum(x == y for a, b in zip(res[0][4], res[0][5]) for x, y in zip(a, b))
    total = sum(len(a) for a in res[0][4])
    assert same >= total - 2, (res[0][4], res[0][5])
