"""Resume on a changed data-parallel size: a run on 3 CPU (gloo) ranks writes its sharded
optimizer state, then the training continues on 2 ranks and on 1 rank from those shards and must
follow the trajectory of the uninterrupted run (the global batch and its mean gradient are the
same whatever the number of ranks that share it)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

STEPS_BEFORE, STEPS_AFTER, BATCH = 3, 3, 12


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(10, 13), torch.nn.Tanh(), torch.nn.Linear(13, 3))


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(STEPS_BEFORE + STEPS_AFTER, BATCH, 10, generator=g), torch.randn(STEPS_BEFORE + STEPS_AFTER, BATCH, 3, generator=g)


def _train(model, opt, xs, ys, steps, rank, world):
    per = BATCH // world
    for i in steps:
        opt.zero_grad()
        x, y = xs[i, rank * per:(rank + 1) * per], ys[i, rank * per:(rank + 1) * per]
        torch.nn.functional.mse_loss(model(x), y).backward()
        opt.step()


def _worker(rank, world, port, base, mode, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cogito_b200.io.checkpoint import load_dp_optimizer_resharded, load_model, save_dp_optimizer_shard, save_model
        from cogito_b200.parallel.data_parallel import DPFusedAdam
        model = _model()
        xs, ys = _data()
        if mode == "resume":
            load_model(base + ".cog", model)
        opt = DPFusedAdam(model.parameters(), group=dist.group.WORLD, lr=5e-2, weight_decay=0.01, max_grad_norm=1.0,
                          bucket_elems=96 * world)          # bucket boundaries move with the group size
        if mode == "resume":
            old = load_dp_optimizer_resharded(base, opt)
            assert old == 3
        else:
            _train(model, opt, xs, ys, range(STEPS_BEFORE), rank, world)
            save_dp_optimizer_shard(base, opt)
            if rank == 0:
                save_model(base + ".cog", model)
            dist.barrier()
        _train(model, opt, xs, ys, range(STEPS_BEFORE, STEPS_BEFORE + STEPS_AFTER), rank, world)
        if rank == 0:
            q.put(torch.cat([p.detach().reshape(-1) for p in model.parameters()]))
    finally:
        dist.destroy_process_group()


def _spawn(world, base, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, base, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


@pytest.mark.timeout(600)
def test_resume_on_fewer_ranks_follows_the_uninterrupted_run(tmp_path):
    base = str(tmp_path / "run")
    full = _spawn(3, base, "first")                     # 3 ranks, uninterrupted; shards written after step 3
    assert len([f for f in os.listdir(tmp_path) if ".opt.dp" in f]) == 3
    two = _spawn(2, base, "resume")                     # one rank lost
    torch.testing.assert_close(two, full, rtol=1e-5, atol=1e-6)
    # a single process without a group
    from cogito_b200.io.checkpoint import load_dp_optimizer_resharded, load_model
    from cogito_b200.parallel.data_parallel import DPFusedAdam
    model = _model()
    load_model(base + ".cog", model)
    opt = DPFusedAdam(model.parameters(), group=None, lr=5e-2, weight_decay=0.01, max_grad_norm=1.0)
    assert load_dp_optimizer_resharded(base, opt) == 3
    xs, ys = _data()
    _train(model, opt, xs, ys, range(STEPS_BEFORE, STEPS_BEFORE + STEPS_AFTER), 0, 1)
    one = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    torch.testing.assert_close(one, full, rtol=1e-5, atol=1e-6)
    # and the shards really mattered: fresh moments give another trajectory
    model2 = _model()
    load_model(base + ".cog", model2)
    opt2 = DPFusedAdam(model2.parameters(), group=None, lr=5e-2, weight_decay=0.01, max_grad_norm=1.0)
    _train(model2, opt2, xs, ys, range(STEPS_BEFORE, STEPS_BEFORE + STEPS_AFTER), 0, 1)
    cold = torch.cat([p.detach().reshape(-1) for p in model2.parameters()])
    assert (cold - full).abs().max() > 1e-3
