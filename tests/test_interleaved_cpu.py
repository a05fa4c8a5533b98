"""Interleaved (virtual-stage) 1F1B: program equals the C generator, the timetable is valid and shrinks
the bubble, and the tick-synchronous executor reproduces single-process gradients on CPU ranks."""
import ctypes
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cogito_b200.parallel.interleaved import InterleavedExecutor, interleaved_1f1b, timetable
from cogito_b200.parallel.pipeline import BACKWARD, FORWARD


def test_program_equals_the_c_generator():
    from capi_defs import L
    lib = L()
    for S, V, M in ((2, 2, 4), (4, 2, 8), (2, 3, 2), (1, 2, 3), (4, 1, 4)):
        for rank in range(S):
            n = ctypes.c_int()
            steps = lib.cg_pipeline_gen_interleaved_stage(S, V, M, rank, ctypes.byref(n))
            c = [(steps[i].action, steps[i].microbatch_id, steps[i].stage_id) for i in range(n.value)]
            py = [(s.action, s.microbatch, s.stage) for s in interleaved_1f1b(S, V, M, rank)]
            assert c == py, (S, V, M, rank)
            ctypes.CDLL(None).free(ctypes.cast(steps, ctypes.c_void_p))
    with pytest.raises(ValueError):
        interleaved_1f1b(4, 2, 6, 0)                    # micro-batches not a multiple of the ranks


def test_timetable_runs_every_compute_once_and_shrinks_the_bubble():
    S, M = 4, 8
    lengths = {}
    for V in (1, 2, 4):
        ticks = timetable(S, V, M)
        seen = [k for now in ticks for k in now.values()]
        assert len(seen) == len(set(seen)) == 2 * M * S * V
        for t, now in enumerate(ticks):                  # a forward never runs before the stage below it
            for action, m, vs in now.values():
                if action == FORWARD and vs > 0:
                    assert any((FORWARD, m, vs - 1) in e.values() for e in ticks[:t])
        lengths[V] = len(ticks) / V                      # one tick is 1/V of a full stage's work
    assert lengths[4] < lengths[2] < lengths[1]
    assert lengths[1] == 2 * (M + S - 1)                 # plain 1F1B: (S - 1) bubble slots each way


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, S, V, M, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=S)
    try:
        torch.manual_seed(0)
        W, B = 16, 3
        layers = [torch.nn.Linear(W, W) for _ in range(S * V)]            # same weights on every rank (same seed)
        xs = [torch.randn(B, W) for _ in range(M)]
        ys = [torch.randn(B, W) for _ in range(M)]
        last = S * V - 1

        def make(c):
            vs = c * S + rank
            lin = layers[vs]

            def fn(x, m):
                h = torch.tanh(lin(x))
                return ((h - ys[m]) ** 2).mean() / M if vs == last else h
            return fn

        ex = InterleavedExecutor(rank, list(range(S)), V, M, (B, W), torch.float32, "cpu")
        loss = ex.run([make(c) for c in range(V)], xs)
        mine = {vs: layers[vs].weight.grad.clone() for vs in range(rank, S * V, S)}
        # single-process oracle on fresh copies
        torch.manual_seed(0)
        ref_layers = [torch.nn.Linear(W, W) for _ in range(S * V)]
        total = 0.0
        for m in range(M):
            h = xs[m]
            for lin in ref_layers:
                h = torch.tanh(lin(h))
            l = ((h - ys[m]) ** 2).mean() / M
            l.backward()
            total += float(l)
        err = max(float((mine[vs] - ref_layers[vs].weight.grad).abs().max()) for vs in mine)
        q.put((rank, None if loss is None else float(loss) * M, total, err, ex.p2p_bytes, ex.bubble_fraction()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("S,V,M", [(2, 2, 4), (4, 2, 4), (2, 3, 2)])
def test_executor_matches_single_process_gradients(S, V, M):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, S, V, M, port, q)) for r in range(S)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, loss, total, err, nbytes, bubble in res:
        assert err < 1e-5, (rank, err)
        assert nbytes > 0 and 0.0 <= bubble < 1.0
        if rank == S - 1:
            assert abs(loss - total) < 1e-5 * max(1.0, abs(total))      # mean of the scaled losses x M = their sum
        else:
            assert loss is None
