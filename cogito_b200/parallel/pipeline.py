"""Pipeline parallelism: the 1F1B schedule and its executor over point-to-point transfers.

``one_f_one_b`` generates one stage's program (S-1-stage warm-up forwards, steady
one-forward/one-backward, cool-down backwards), the same program as
``cg_pipeline_gen_1f1b_stage`` of the host library (reference: cg_schedule_action /
cg_schedule_step / cg_pipeline_gen_1f1b, include/cg_pipeline.h:27-40,78-93; the reference
generator only produces stage 0 and its executor ``cg_pipeline_forward_backward`` is declared
only, src/pipeline/pipeline.c).

Transfers are NCCL (or gloo) point-to-point calls.  A send that is directly followed by a
receive in the program is posted together with it as one batch, which is what keeps two
neighbouring stages in steady state (one sending forward while the other sends backward) from
waiting on each other's queues.  With tensor parallelism inside a stage the residual stream is
sequence-sharded, so rank (tp=i) of one stage talks only to rank (tp=i) of the next and moves
1/tp of the activation.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

FORWARD, BACKWARD, SEND_FWD, RECV_FWD, SEND_BWD, RECV_BWD, OPTIMIZER = range(7)


@dataclass(frozen=True)
class Step:
    action: int
    microbatch: int
    stage: int


def one_f_one_b(num_stages: int, num_microbatches: int, stage: int) -> list[Step]:
    S, M = num_stages, num_microbatches
    if not (S > 0 and M > 0 and 0 <= stage < S):
        raise ValueError("bad pipeline shape")
    out: list[Step] = []

    def fwd(m):
        if stage != 0:
            out.append(Step(RECV_FWD, m, stage))
        out.append(Step(FORWARD, m, stage))
        if stage != S - 1:
            out.append(Step(SEND_FWD, m, stage))

    def bwd(m):
        if stage != S - 1:
            out.append(Step(RECV_BWD, m, stage))
        out.append(Step(BACKWARD, m, stage))
        if stage != 0:
            out.append(Step(SEND_BWD, m, stage))

    warm = min(S - 1 - stage, M)
    f = b = 0
    while f < warm:
        fwd(f); f += 1
    while f < M:
        fwd(f); f += 1
        bwd(b); b += 1
    while b < M:
        bwd(b); b += 1
    out.append(Step(OPTIMIZER, -1, stage))
    return out


class PipelineExecutor:
    """Runs one training step of one pipeline stage.

    stage_fn(x_or_ids, microbatch) -> activation (or the loss on the last stage);
    first stage receives the micro-batch's token ids, later stages the received activation.
    """

    def __init__(self, stage: int, num_stages: int, num_microbatches: int, prev_rank: int | None, next_rank: int | None,
                 act_shape, act_dtype, device, group=None):
        self.stage, self.S, self.M = stage, num_stages, num_microbatches
        self.prev, self.next = prev_rank, next_rank
        self.shape, self.dtype, self.device = tuple(act_shape), act_dtype, torch.device(device)
        self.group = group
        self.program = one_f_one_b(num_stages, num_microbatches, stage)
        self.p2p_bytes = 0

    # -------------------------------------------------------------- transfers
    def _post(self, ops):
        if not ops:
            return
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    def _send_op(self, t, peer):
        self.p2p_bytes += t.numel() * t.element_size()
        return dist.P2POp(dist.isend, t.contiguous(), peer, self.group)

    def _recv_op(self, peer):
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        return buf, dist.P2POp(dist.irecv, buf, peer, self.group)

    # ------------------------------------------------------------------- step
    def run(self, stage_fn, first_inputs=None):
        """first_inputs[m]: what the first stage feeds micro-batch m (ignored elsewhere).
        On the last stage stage_fn returns the micro-batch loss, built so that its backward is
        already multiplied by loss_scale / M.  Returns the mean loss there, None elsewhere."""
        inputs, outputs = {}, {}
        grads_in = {}
        losses = []
        prog = self.program
        i = 0
        pending_recv = None            # (kind, microbatch, buffer) posted together with the previous send
        while i < len(prog):
            st = prog[i]
            m = st.microbatch
            if st.action in (RECV_FWD, RECV_BWD):
                if pending_recv is not None and pending_recv[:2] == (st.action, m):
                    buf = pending_recv[2]
                    pending_recv = None
                else:
                    buf, op = self._recv_op(self.prev if st.action == RECV_FWD else self.next)
                    self._post([op])
                if st.action == RECV_FWD:
                    inputs[m] = buf.requires_grad_(True)
                else:
                    grads_in[m] = buf
            elif st.action == FORWARD:
                x = first_inputs[m] if self.stage == 0 else inputs[m]
                y = stage_fn(x, m)
                outputs[m] = y
                if self.stage == self.S - 1:
                    losses.append(y.detach().float())
            elif st.action == BACKWARD:
                y = outputs.pop(m)
                if self.stage == self.S - 1:
                    y.backward()       # stage_fn built the loss with grad_scale = loss_scale / M
                else:
                    y.backward(grads_in.pop(m))
            elif st.action in (SEND_FWD, SEND_BWD):
                if st.action == SEND_FWD:
                    t, peer = outputs[m].detach(), self.next
                else:
                    t, peer = inputs.pop(m).grad, self.prev
                ops = [self._send_op(t, peer)]
                nxt = prog[i + 1] if i + 1 < len(prog) else None
                if nxt is not None and nxt.action in (RECV_FWD, RECV_BWD):
                    buf, rop = self._recv_op(self.prev if nxt.action == RECV_FWD else self.next)
                    ops.append(rop)
                    pending_recv = (nxt.action, nxt.microbatch, buf)
                self._post(ops)
            i += 1
        if self.stage == self.S - 1:
            return torch.stack(losses).mean()
        return None

    def bubble_fraction(self) -> float:
        """Idle share of the schedule: (S - 1) / (M + S - 1)."""
        return (self.S - 1) / (self.M + self.S - 1)
