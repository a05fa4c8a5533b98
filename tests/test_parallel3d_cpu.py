"""DP x TP x PP Llama on CPU ranks (gloo): the 1F1B executor, tensor-parallel Llama blocks and
the data-parallel optimizer must reproduce the single-device training trajectory."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cogito_b200.parallel.pipeline import BACKWARD, FORWARD, OPTIMIZER, RECV_FWD, SEND_BWD, SEND_FWD, one_f_one_b


def test_python_schedule_equals_the_c_generator():
    import ctypes
    from capi_defs import L
    lib = L()
    for S, M in ((1, 3), (2, 4), (4, 8), (4, 2), (3, 7)):
        for stage in range(S):
            n = ctypes.c_int()
            steps = lib.cg_pipeline_gen_1f1b_stage(S, M, stage, ctypes.byref(n))
            c = [(steps[i].action, steps[i].microbatch_id, steps[i].stage_id) for i in range(n.value)]
            py = [(s.action, s.microbatch, s.stage) for s in one_f_one_b(S, M, stage)]
            assert c == py
            ctypes.CDLL(None).free(ctypes.cast(steps, ctypes.c_void_p))
    prog = one_f_one_b(4, 8, 1)
    assert [s.action for s in prog[:6]] == [RECV_FWD, FORWARD, SEND_FWD, RECV_FWD, FORWARD, SEND_FWD]
    assert prog[-1].action == OPTIMIZER and sum(s.action == BACKWARD for s in prog) == 8 and sum(s.action == SEND_BWD for s in prog) == 8


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, dp, tp, pp, q, virtual=1, clip=0.0, recompute=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cogito_b200.models.llama import Llama, LlamaConfig
        from cogito_b200.optim.fused import FusedAdam
        from cogito_b200.parallel.groups import init_parallel
        from cogito_b200.parallel.llama_parallel import Trainer3D, shard_llama_state
        from cogito_b200.train import Trainer
        from cogito_b200.utils.rng import manual_seed
        manual_seed(0)
        cfg = LlamaConfig(vocab_size=64, n_layer=4, d_model=32, n_head=4, n_kv_head=2, d_ff=64, max_seq_len=16)
        full = Llama(cfg)
        ctx = init_parallel(dp, tp, pp)
        M, mb, T = 4, 1, 16
        t3 = Trainer3D(cfg, ctx, "cpu", num_microbatches=M, micro_batch=mb, seq_len=T, lr=1e-2, loss_scale=None, max_grad_norm=clip,
                       virtual_stages=virtual, recompute=recompute)
        t3.load_from(full)
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, 64, (dp * M * mb, T), generator=g)
        tg = torch.randint(0, 64, (dp * M * mb, T), generator=g)
        ref = Trainer(full, FusedAdam(full.parameters(), lr=1e-2, max_grad_norm=clip), micro_batch=mb)
        lf = [float(ref.step(ids, tg)) for _ in range(3)]
        d = ctx.coords.dp_rank
        mine_ids, mine_tg = ids[d * M * mb:(d + 1) * M * mb], tg[d * M * mb:(d + 1) * M * mb]
        lt = []
        for _ in range(3):
            loss = t3.step(mine_ids, mine_tg)
            lt.append(None if loss is None else float(loss))
        # the gradients of the last step are still in the flat buffers: the replica-wide sum of squares that
        # the optimizer clips with must equal the single-device one (replicated parameters counted once)
        norm_ref = float((ref.opt.grad.double() ** 2).sum())
        norm_mp = None
        if getattr(t3.opt, "stats_sync", None) is not None:
            f, n2 = torch.zeros(1, dtype=torch.int32), (t3.opt.grad ** 2).sum().reshape(1).clone()
            t3.opt.stats_sync(f, n2)
            norm_mp = float(n2)
        q.put((rank, ctx.coords.dp_rank, ctx.coords.pp_rank, lf, lt, t3.pipe.p2p_bytes, norm_ref, norm_mp,
               getattr(t3.pipe, "max_recvs_in_flight", 0)))
    finally:
        dist.destroy_process_group()


# (1, 2, 2, 2, 0): interleaved 1F1B, 2 chunks per rank; (2, 2, 2, 1, 1): clipping on, so the data-parallel average is an
# all-reduce and the optimizer steps with replica-wide statistics; the last two: activation recomputation per block
# (second forward pass of every block inside backward, tensor-parallel collectives included) and per stage
@pytest.mark.parametrize("dp,tp,pp,virtual,clip,recompute", [(1, 1, 2, 1, 0.0, None), (1, 2, 2, 1, 0.0, None), (2, 2, 2, 1, 0.0, None),
                                                             (1, 2, 2, 2, 0.0, None), (2, 2, 2, 1, 1.0, None),
                                                             (1, 2, 2, 1, 0.0, "block"), (1, 1, 2, 1, 0.0, "stage")])
def test_3d_llama_matches_single_device(dp, tp, pp, virtual, clip, recompute):
    world = dp * tp * pp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, dp, tp, pp, q, virtual, clip, recompute)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    last = [r for r in res if r[2] == pp - 1]
    assert len(last) == dp * tp
    ref = res[0][3]
    assert ref[-1] < ref[0]
    # step 0: each replica's loss is over its own half of the batch; their mean is the full-batch loss
    first = {}
    for rank, d, p_, lf, lt, nbytes, *_ in last:
        first.setdefault(d, lt[0])
        assert nbytes > 0 or pp == 1
    assert abs(sum(first.values()) / len(first) - ref[0]) < 2e-3
    # later steps: parameters stayed in lock-step with the single-device run
    for step in (1, 2):
        vals = {}
        for rank, d, p_, lf, lt, nbytes, *_ in last:
            vals.setdefault(d, lt[step])
        assert abs(sum(vals.values()) / len(vals) - ref[step]) < 3e-3, (step, vals, ref)
    if pp > 1 and virtual == 1:
        # receives were posted ahead of the pass that needs them: at some point two were in flight on a middle or
        # last stage (the next forward input and the next gradient)
        assert max(r[8] for r in res) >= 1
    for r in res:
        if r[2] != pp - 1:
            assert all(v is None for v in r[4])
        if dp == 1 or clip > 0:
            assert r[7] is not None and abs(r[7] - r[6]) < 5e-3 * r[6], (r[6], r[7])
