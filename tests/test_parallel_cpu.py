"""Multi-rank logic on CPU ranks (gloo): rank arithmetic, process groups, tensor-parallel
GPT-2 equivalence with the single-device model."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cogito_b200.parallel.groups import Coords, group_ranks, rank_of


def test_rank_mapping_matches_reference_arithmetic():
    dp, tp, pp = 2, 2, 2
    seen = set()
    for r in range(8):
        c = Coords(r, dp, tp, pp)
        assert c.tp_rank == r % tp and c.pp_rank == (r // tp) % pp and c.dp_rank == r // (tp * pp)
        assert rank_of(c.dp_rank, c.pp_rank, c.tp_rank, tp, pp) == r
        assert c.tp_color() == c.dp_rank * pp + c.pp_rank
        assert c.pp_color() == c.dp_rank * tp + c.tp_rank
        assert c.dp_color() == c.pp_rank * tp + c.tp_rank
        seen.add((c.dp_rank, c.pp_rank, c.tp_rank))
    assert len(seen) == 8
    tpg, ppg, dpg = group_ranks(8, dp, tp, pp)
    assert sorted(map(tuple, tpg.values())) == [(0, 1), (2, 3), (4, 5), (6, 7)]
    assert sorted(map(tuple, ppg.values())) == [(0, 2), (1, 3), (4, 6), (5, 7)]
    assert sorted(map(tuple, dpg.values())) == [(0, 4), (1, 5), (2, 6), (3, 7)]
    with pytest.raises(ValueError):
        group_ranks(8, 2, 2, 3)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tp_worker(rank, world, port, q, heads=4):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cogito_b200.models.gpt2 import GPT2, GPT2Config
        from cogito_b200.optim.fused import FusedAdam
        from cogito_b200.parallel.tensor_parallel import build_tp_gpt2, shard_gpt2_state
        from cogito_b200.train import Trainer
        from cogito_b200.utils.rng import manual_seed
        manual_seed(0)
        cfg = GPT2Config(vocab_size=64, n_layer=2, d_model=8 * heads, n_head=heads, d_ff=64, max_seq_len=16)
        full = GPT2(cfg)
        tp, sync = build_tp_gpt2(cfg, rank, world, "cpu", dist.group.WORLD, micro_tokens=64)
        shard_gpt2_state(full, tp)
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, 64, (4, 16), generator=g)
        tg = torch.randint(0, 64, (4, 16), generator=g)
        of = FusedAdam(full.parameters(), lr=1e-2)
        ot = FusedAdam(tp._ordered, lr=1e-2)
        sync.attach(ot)
        tf = Trainer(full, of, micro_batch=4)
        tt = Trainer(tp, ot, micro_batch=4, parallel=sync)
        lf = [float(tf.step(ids, tg)) for _ in range(4)]
        lt = [float(tt.step(ids, tg)) for _ in range(4)]
        q.put((rank, lf, lt))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 3])        # 3 heads over 2 ranks: one rank holds two, the other one
def test_tensor_parallel_gpt2_matches_single_device_on_two_cpu_ranks(heads):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q, heads)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, lf, lt in res:
        assert lf[-1] < lf[0]
        for a, b in zip(lf, lt):
            assert abs(a - b) < 2e-3, (rank, lf, lt)


def _dp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cogito_b200.optim.fused import FusedAdam
        from cogito_b200.parallel.data_parallel import DPFusedAdam
        from cogito_b200 import nn as cnn
        from cogito_b200.ops import loss as L
        from cogito_b200.utils.rng import manual_seed
        manual_seed(0)
        mk = lambda: cnn.Sequential(cnn.Linear(12, 16, act="relu"), cnn.Linear(16, 4))
        ref, dp = mk(), mk()
        dp.load_state_dict(ref.state_dict())
        o_ref = FusedAdam(ref.parameters(), lr=1e-2, master_weights=False)
        o_dp = DPFusedAdam(dp.parameters(), dist.group.WORLD, lr=1e-2, bucket_elems=64)    # several buckets, the last one short
        assert o_dp.nbuckets > 2 and sum(c for _, c, _ in o_dp.segments) == o_dp.n // world
        g = torch.Generator().manual_seed(3)
        X = torch.randn(8, 12, generator=g)
        Y = torch.randint(0, 4, (8,), generator=g)
        for _ in range(5):
            o_ref.zero_grad(); o_dp.zero_grad()
            L.softmax_cross_entropy_small(ref(X), Y).backward()
            half = slice(rank * 4, rank * 4 + 4)
            L.softmax_cross_entropy_small(dp(X[half]), Y[half]).backward()
            o_ref.step(); o_dp.step()
        diff = max(float((a - b).abs().max()) for a, b in zip(ref.parameters(), dp.parameters()))
        q.put((rank, diff))
    finally:
        dist.destroy_process_group()


def test_dp_fused_adam_matches_full_batch_on_two_cpu_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, diff in res:
        assert diff < 1e-5, (rank, diff)


def _torch_tp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import types
        from cogito_b200 import bench_support as bs
        from cogito_b200.models.gpt2 import GPT2Config
        torch.manual_seed(0)
        cfg = GPT2Config(vocab_size=64, n_layer=2, d_model=32, n_head=4, d_ff=64, max_seq_len=16)
        # one unsplit model; every rank cuts its shard out of it
        ref = bs._TorchTPGPT2(cfg, 0, 1, None)
        tp = bs._TorchTPGPT2(cfg, rank, world, dist.group.WORLD)
        hd, hl, fl, vl = 8, 4 // world, 64 // world, 64 // world
        with torch.no_grad():
            tp.wte.copy_(ref.wte[rank * vl:(rank + 1) * vl]); tp.wpe.copy_(ref.wpe)
            for a, b in zip(ref.blocks, tp.blocks):
                wq = a.qkv.weight.view(3, 4, hd, 32)[:, rank * hl:(rank + 1) * hl]
                b.qkv.weight.copy_(wq.reshape(3 * hl * hd, 32))
                b.qkv.bias.copy_(a.qkv.bias.view(3, 4, hd)[:, rank * hl:(rank + 1) * hl].reshape(-1))
                b.proj.weight.copy_(a.proj.weight[:, rank * hl * hd:(rank + 1) * hl * hd])
                b.up.weight.copy_(a.up.weight[rank * fl:(rank + 1) * fl]); b.up.bias.copy_(a.up.bias[rank * fl:(rank + 1) * fl])
                b.down.weight.copy_(a.down.weight[:, rank * fl:(rank + 1) * fl])
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, 64, (4, 16), generator=g)
        tg = torch.randint(0, 64, (4, 16), generator=g)
        l_ref, l_tp = ref(ids, tg), tp(ids, tg)
        l_ref.backward(); l_tp.backward()
        gq_ref = ref.blocks[0].qkv.weight.grad.view(3, 4, hd, 32)[:, rank * hl:(rank + 1) * hl].reshape(3 * hl * hd, 32)
        q.put((rank, float(l_ref), float(l_tp), float((gq_ref - tp.blocks[0].qkv.weight.grad).abs().max()),
               float(gq_ref.abs().max())))
    finally:
        dist.destroy_process_group()


def test_torch_tensor_parallel_baseline_of_the_bench_matches_its_unsplit_form():
    """The comparison arm of bench.py (NCCL-style collectives + library GEMMs) computes the same
    loss and gradients as the same model on one rank."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_torch_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(30)
    for rank, l_ref, l_tp, gerr, gmax in res:
        assert abs(l_ref - l_tp) < 1e-4 * max(1.0, abs(l_ref)), res
        assert gerr < 1e-4 * max(gmax, 1e-3), res
