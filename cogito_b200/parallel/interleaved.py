"""Interleaved (virtual-stage) 1F1B: every pipeline rank holds V model chunks, virtual stage
``chunk * S + rank``, which shrinks the pipeline bubble by V at the price of V times more transfers.

``interleaved_1f1b`` is the per-rank program, the same as ``cg_pipeline_gen_interleaved_stage`` of the
host library (the reference declares no such schedule: its generator, src/pipeline/pipeline.c:38-80,
produces plain 1F1B for stage 0 only; virtual stages are listed as missing in its header comments).

The executor is tick-synchronous.  Every rank simulates the whole pipeline from the programs (each
compute takes one tick and starts once its input was produced in an earlier tick), which gives each rank
the same global timetable.  After tick t every rank posts, as ONE batch of point-to-point operations,
the sends of what it produced in tick t and the receives of what its neighbours produced in tick t for
it, both sides listing the transfers of a pair in the same canonical order.  All ranks move through the
ticks together, a rank only ever waits for batches of the same tick, and a batch is one NCCL group (or
tagged gloo messages), so the wrap-around transfers of the interleaved schedule (last rank -> first rank,
and with two ranks both directions between the same pair) cannot deadlock or be mismatched.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .pipeline import BACKWARD, FORWARD, OPTIMIZER, RECV_BWD, RECV_FWD, SEND_BWD, SEND_FWD, Step


def interleaved_1f1b(num_ranks: int, chunks: int, num_microbatches: int, rank: int) -> list[Step]:
    """Program of pipeline rank ``rank``; ``Step.stage`` carries the virtual stage chunk * S + rank.
    The number of micro-batches must be a multiple of the number of ranks."""
    S, V, M = num_ranks, chunks, num_microbatches
    if not (S > 0 and V > 0 and M > 0 and 0 <= rank < S) or M % S:
        raise ValueError("bad interleaved pipeline shape (micro-batches must be a multiple of the ranks)")
    total, last = M * V, S * V - 1
    warm = min((S - rank - 1) * 2 + (V - 1) * S, total)
    out: list[Step] = []

    def chunk_of(k, fwd):
        c = (k // S) % V
        return c if fwd else V - 1 - c

    def mb_of(k):
        return (k // (S * V)) * S + k % S

    def do_f(k):
        vs, m = chunk_of(k, True) * S + rank, mb_of(k)
        if vs != 0:
            out.append(Step(RECV_FWD, m, vs))
        out.append(Step(FORWARD, m, vs))
        if vs != last:
            out.append(Step(SEND_FWD, m, vs))

    def do_b(k):
        vs, m = chunk_of(k, False) * S + rank, mb_of(k)
        if vs != last:
            out.append(Step(RECV_BWD, m, vs))
        out.append(Step(BACKWARD, m, vs))
        if vs != 0:
            out.append(Step(SEND_BWD, m, vs))

    f = b = 0
    while f < warm:
        do_f(f); f += 1
    while f < total:
        do_f(f); f += 1
        do_b(b); b += 1
    while b < total:
        do_b(b); b += 1
    out.append(Step(OPTIMIZER, -1, rank))
    return out


def timetable(num_ranks: int, chunks: int, num_microbatches: int):
    """Simulates all ranks.  Returns ``ticks``: a list over time of {rank: (action, microbatch, virtual
    stage)} for the computes that run in that tick.  Raises if the programs cannot make progress."""
    S, V, M = num_ranks, chunks, num_microbatches
    last = S * V - 1
    progs = [[s for s in interleaved_1f1b(S, V, M, r) if s.action in (FORWARD, BACKWARD)] for r in range(S)]
    pos = [0] * S
    done_at: dict = {}
    ticks = []
    remaining = sum(len(p) for p in progs)
    t = 0
    while remaining:
        now = {}
        for r in range(S):
            if pos[r] == len(progs[r]):
                continue
            st = progs[r][pos[r]]
            if st.action == FORWARD:
                dep = None if st.stage == 0 else (FORWARD, st.microbatch, st.stage - 1)
            else:
                dep = (FORWARD, st.microbatch, st.stage) if st.stage == last else (BACKWARD, st.microbatch, st.stage + 1)
            if dep is None or done_at.get(dep, t) < t:
                now[r] = (st.action, st.microbatch, st.stage)
        if not now:
            raise RuntimeError("interleaved schedule cannot make progress")
        for r, key in now.items():
            done_at[key] = t
            pos[r] += 1
            remaining -= 1
        ticks.append(now)
        t += 1
    return ticks


class InterleavedExecutor:
    """One training step of one pipeline rank that holds ``chunks`` model chunks.

    ring: global ranks of the pipeline group in stage order (ring[i] holds virtual stages i, i + S, ...).
    stage_fns[c](x, microbatch) runs chunk c: the first virtual stage gets first_inputs[microbatch],
    the last one returns the micro-batch loss (built so that its backward already carries
    loss_scale / M), every other one maps an activation of ``act_shape`` to the next."""

    def __init__(self, rank_in_ring: int, ring: list[int], chunks: int, num_microbatches: int, act_shape, act_dtype, device, group=None):
        self.r, self.ring, self.S, self.V, self.M = rank_in_ring, list(ring), len(ring), chunks, num_microbatches
        self.shape, self.dtype, self.device, self.group = tuple(act_shape), act_dtype, torch.device(device), group
        self.ticks = timetable(self.S, chunks, num_microbatches)
        self.last = self.S * chunks - 1
        self.p2p_bytes = 0
        self.tagged = dist.is_initialized() and dist.get_backend(group) == "gloo"

    def _dest(self, action, vs):
        """Pipeline rank that consumes the output of (action, vs), or None."""
        if action == FORWARD:
            return None if vs == self.last else (vs + 1) % self.S
        return None if vs == 0 else (vs - 1) % self.S

    def bubble_fraction(self) -> float:
        """Idle share of this rank in the simulated timetable."""
        busy = sum(1 for now in self.ticks if self.r in now)
        return 1.0 - busy / len(self.ticks)

    def run(self, stage_fns, first_inputs):
        inbox, saved, losses = {}, {}, []
        for now in self.ticks:
            mine = now.get(self.r)
            produced = None
            if mine is not None:
                action, m, vs = mine
                c = vs // self.S
                if action == FORWARD:
                    x = first_inputs[m] if vs == 0 else inbox.pop((FORWARD, m, vs)).requires_grad_(True)
                    y = stage_fns[c](x, m)
                    saved[(m, vs)] = (x, y)
                    if vs == self.last:
                        losses.append(y.detach().float())
                    else:
                        produced = y.detach()
                else:
                    x, y = saved.pop((m, vs))
                    if vs == self.last:
                        y.backward()
                    else:
                        y.backward(inbox.pop((BACKWARD, m, vs)))
                    if vs != 0:
                        produced = x.grad
            # transfers of this tick, per peer in the canonical order (action, microbatch, virtual stage)
            ops, recvs = [], []
            for src in sorted(now):
                action, m, vs = now[src]
                dst = self._dest(action, vs)
                if dst is None:
                    continue
                key = (action, m, vs + 1 if action == FORWARD else vs - 1)       # what the consumer calls it
                tag = (0 if action == FORWARD else 1 << 20) + key[2] * 1024 + m if self.tagged else 0
                if src == self.r and dst == self.r:
                    inbox[key] = produced                                        # one rank: the chunk hands over to itself
                elif src == self.r:
                    t = produced.contiguous()
                    self.p2p_bytes += t.numel() * t.element_size()
                    ops.append(((dst, 0) + key, dist.P2POp(dist.isend, t, self.ring[dst], self.group, tag)))
                elif dst == self.r:
                    buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
                    ops.append(((src, 1) + key, dist.P2POp(dist.irecv, buf, self.ring[src], self.group, tag)))
                    recvs.append((key, buf))
            if ops:
                ops.sort(key=lambda o: o[0])
                for w in dist.batch_isend_irecv([o for _, o in ops]):
                    w.wait()
                for key, buf in recvs:
                    inbox[key] = buf
        return torch.stack(losses).mean() if losses else None
